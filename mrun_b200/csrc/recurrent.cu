// Mixers that carry a state of fixed size from token to token, and the short causal convolutions
// in front of them.
//
// A step's tokens come as segments (one per request: rows seg_q_start[s] .. seg_q_start[s+1] of
// the flat batch, state slot seg_slot[s]); a segment of zero rows is padding.  Every kernel reads
// the state its request left, walks the segment's tokens in order and leaves the state for the
// next step, so a token's result does not depend on how the request was cut into steps or on the
// requests beside it.  States and all arithmetic of the recurrences are 32-bit.
//
// Kernels:
//   causal_conv     y_t = sum_j w[:, j] x_(t - taps + 1 + j) per channel (the last tap meets the
//                   token itself; zeros before the sequence's start), either added to x_t or
//                   passed through SiLU; the last taps - 1 inputs of a request are its state
//   decay_scan      per head S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t (linear attention
//                   with one decay a head; q, k, v optionally through SiLU on the way in)
//   delta_scan      per head, with a decay per key channel g = exp(-exp(A_h) softplus(a + bias)),
//                   a write strength beta = sigmoid(b) and unit-length q (times dim^-1/2) and k:
//                   S <- g * S (rows); u = beta (v - S^T k); S <- S + k u^T; o = S^T q
//   gated_norm      per group of n outputs: o / sqrt(mean(o^2) + eps) * w * sigmoid(gate)
#include "common.cuh"

using namespace mrun;

namespace {

constexpr int MAX_TAPS = 8;
constexpr int CONV_TILE = 64;       // tokens a block walks; at least MAX_TAPS - 1

template <bool EXACT> __device__ __forceinline__ float silu_f(float z) {
    if constexpr (EXACT) return z / (1.f + expf(-z));
    else return __fdividef(z, 1.f + __expf(-z));
}

// grid (channel chunks, token tiles, segments); a thread a channel.  Only a segment's first tile
// reads the state (its tokens have fewer than taps - 1 tokens of the step before them), and that
// block also leaves the new state once it has read the old one.
template <typename TA>
__global__ void __launch_bounds__(128)
causal_conv_kernel(const TA* __restrict__ x, long ldx, const float* __restrict__ w, TA* __restrict__ state,
                   TA* __restrict__ out, long ldo, const int* __restrict__ seg_q_start,
                   const int* __restrict__ seg_slot, int C, int taps, int residual, int silu) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int seg = blockIdx.z;
    const int q0 = seg_q_start[seg], n = seg_q_start[seg + 1] - q0;
    const int l0 = blockIdx.y * CONV_TILE;
    if (c >= C || l0 >= n) return;
    TA* st = state + (size_t)seg_slot[seg] * (taps - 1) * C + c;
    float wv[MAX_TAPS], hist[MAX_TAPS - 1];      // hist[j - 1]: the input j tokens back
#pragma unroll
    for (int j = 0; j < MAX_TAPS; ++j) wv[j] = j < taps ? w[(size_t)c * taps + j] : 0.f;
#pragma unroll
    for (int j = 1; j < MAX_TAPS; ++j) {
        hist[j - 1] = 0.f;
        if (j < taps) {
            const int l = l0 - j;
            hist[j - 1] = l >= 0 ? to_float(x[(size_t)(q0 + l) * ldx + c]) : to_float(st[(size_t)(l + taps - 1) * C]);
        }
    }
    const int end = min(n, l0 + CONV_TILE);
    for (int l = l0; l < end; ++l) {
        const float cur = to_float(x[(size_t)(q0 + l) * ldx + c]);
        float acc = 0.f;
#pragma unroll
        for (int j = MAX_TAPS - 1; j >= 1; --j)          // oldest input first
            if (j < taps) acc = fmaf(wv[taps - 1 - j], hist[j - 1], acc);
        acc = fmaf(wv[taps - 1], cur, acc);
        float y = residual ? cur + acc : acc;
        if (silu) y = silu_f<true>(y);
        out[(size_t)(q0 + l) * ldo + c] = from_float<TA>(y);
#pragma unroll
        for (int j = MAX_TAPS - 1; j >= 2; --j) hist[j - 1] = hist[j - 2];
        hist[0] = cur;
    }
    if (blockIdx.y == 0) {
        float fresh[MAX_TAPS - 1];
#pragma unroll
        for (int i = 0; i < MAX_TAPS - 1; ++i) {
            fresh[i] = 0.f;
            if (i < taps - 1) {
                const int l = n - (taps - 1) + i;
                fresh[i] = l >= 0 ? to_float(x[(size_t)(q0 + l) * ldx + c]) : to_float(st[(size_t)(l + taps - 1) * C]);
            }
        }
#pragma unroll
        for (int i = 0; i < MAX_TAPS - 1; ++i)
            if (i < taps - 1) st[(size_t)i * C] = from_float<TA>(fresh[i]);
    }
}

// ------------------------------------------------------------------------------------------
// The scans.  grid (value-column chunks of 32, heads, segments), block (32, DS): lane j owns
// column j of the head's state, slice r the key rows r * DPT .. of it, DPT of them in registers.
// The segment's tokens are staged TOKENS at a time into shared memory (q, k, the decays, the
// block's 32 values, the write strengths), then walked one by one.  With DS > 1 the partial sums
// of the slices meet in shared memory and are added in slice order.
// ------------------------------------------------------------------------------------------
constexpr int SCAN_TOKENS = 8;

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

template <typename TA, int DPT, bool DELTA>
__global__ void __launch_bounds__(64)
scan_kernel(const TA* __restrict__ q, const TA* __restrict__ k, const TA* __restrict__ v, long ld, int group,
            const float* __restrict__ a, const TA* __restrict__ b, long ldb, const float* __restrict__ a_log,
            const float* __restrict__ dt_bias, const float* __restrict__ decay, float* __restrict__ state,
            float* __restrict__ out, const int* __restrict__ seg_q_start, const int* __restrict__ seg_slot,
            int H, int D, int V, int silu_inputs) {
    extern __shared__ float smem[];
    const int lane = threadIdx.x, slice = threadIdx.y, DS = blockDim.y;
    const int tid = slice * 32 + lane, nthreads = 32 * DS;
    const int h = blockIdx.y, seg = blockIdx.z;
    const int q0 = seg_q_start[seg], n = seg_q_start[seg + 1] - q0;
    if (n <= 0) return;
    const int col = blockIdx.x * 32 + lane;
    const bool live = col < V;
    const int kh = h / group;                    // the q/k head this head reads
    float* qs = smem;                            // [SCAN_TOKENS][D]
    float* ks = qs + SCAN_TOKENS * D;
    float* gs = ks + SCAN_TOKENS * D;            // [SCAN_TOKENS][D] (DELTA)
    float* vs = gs + (DELTA ? SCAN_TOKENS * D : 0);   // [SCAN_TOKENS][32]
    float* bs = vs + SCAN_TOKENS * 32;           // [SCAN_TOKENS]
    float* red = bs + SCAN_TOKENS;               // [DS][32]

    float S[DPT];
    float* st = state + (((size_t)seg_slot[seg] * H + h) * D) * V + col;
    const int row0 = slice * DPT;
#pragma unroll
    for (int i = 0; i < DPT; ++i) S[i] = (live && row0 + i < D) ? st[(size_t)(row0 + i) * V] : 0.f;
    const float head_decay = DELTA ? 0.f : decay[h];
    const float rate = DELTA ? expf(a_log[h]) : 0.f;
    const float q_scale = DELTA ? rsqrtf((float)D) : 1.f;

    for (int t0 = 0; t0 < n; t0 += SCAN_TOKENS) {
        const int m = min(SCAN_TOKENS, n - t0);
        __syncthreads();
        for (int e = tid; e < m * D; e += nthreads) {
            const int tt = e / D, i = e - tt * D;
            const size_t row = (size_t)(q0 + t0 + tt);
            float qv = to_float(q[row * ld + (size_t)kh * D + i]);
            float kv = to_float(k[row * ld + (size_t)kh * D + i]);
            if (silu_inputs) { qv = silu_f<true>(qv); kv = silu_f<true>(kv); }
            qs[tt * D + i] = qv;
            ks[tt * D + i] = kv;
            if constexpr (DELTA) {
                const float step = softplus_f(a[row * ((size_t)H * D) + (size_t)h * D + i] + dt_bias[(size_t)h * D + i]);
                gs[tt * D + i] = expf(-rate * step);
            }
        }
        for (int e = tid; e < m * 32; e += nthreads) {
            const int tt = e >> 5, j = e & 31;
            const int cj = blockIdx.x * 32 + j;
            float vv = cj < V ? to_float(v[(size_t)(q0 + t0 + tt) * ld + (size_t)h * V + cj]) : 0.f;
            if (silu_inputs) vv = silu_f<true>(vv);
            vs[e] = vv;
        }
        if constexpr (DELTA) {
            if (tid < m) bs[tid] = 1.f / (1.f + expf(-to_float(b[(size_t)(q0 + t0 + tid) * ldb + h])));
            __syncthreads();
            // unit length per head: a warp a token
            for (int tt = slice; tt < m; tt += DS) {
                float sq = 0.f, sk = 0.f;
                for (int i = lane; i < D; i += 32) {
                    sq = fmaf(qs[tt * D + i], qs[tt * D + i], sq);
                    sk = fmaf(ks[tt * D + i], ks[tt * D + i], sk);
                }
                sq = warp_sum(sq); sk = warp_sum(sk);
                const float fq = q_scale / sqrtf(sq + 1e-6f), fk = 1.f / sqrtf(sk + 1e-6f);
                for (int i = lane; i < D; i += 32) { qs[tt * D + i] *= fq; ks[tt * D + i] *= fk; }
            }
        }
        __syncthreads();
        for (int tt = 0; tt < m; ++tt) {
            const float* qt = qs + tt * D + row0;
            const float* kt = ks + tt * D + row0;
            const float vv = vs[tt * 32 + lane];
            float o = 0.f;
            if constexpr (DELTA) {
                const float* gt = gs + tt * D + row0;
                float kv = 0.f;
#pragma unroll
                for (int i = 0; i < DPT; ++i)
                    if (row0 + i < D) { S[i] *= gt[i]; kv = fmaf(S[i], kt[i], kv); }
                if (DS > 1) {
                    red[slice * 32 + lane] = kv;
                    __syncthreads();
                    kv = 0.f;
                    for (int r = 0; r < DS; ++r) kv += red[r * 32 + lane];
                    __syncthreads();
                }
                const float u = bs[tt] * (vv - kv);
#pragma unroll
                for (int i = 0; i < DPT; ++i)
                    if (row0 + i < D) { S[i] = fmaf(kt[i], u, S[i]); o = fmaf(S[i], qt[i], o); }
            } else {
#pragma unroll
                for (int i = 0; i < DPT; ++i)
                    if (row0 + i < D) { S[i] = fmaf(head_decay, S[i], kt[i] * vv); o = fmaf(S[i], qt[i], o); }
            }
            if (DS > 1) {
                red[slice * 32 + lane] = o;
                __syncthreads();
                o = 0.f;
                for (int r = 0; r < DS; ++r) o += red[r * 32 + lane];
                __syncthreads();
            }
            if (live && slice == 0) out[(size_t)(q0 + t0 + tt) * ((size_t)H * V) + (size_t)h * V + col] = o;
        }
    }
#pragma unroll
    for (int i = 0; i < DPT; ++i)
        if (live && row0 + i < D) st[(size_t)(row0 + i) * V] = S[i];
}

// A warp a (token, group).
template <typename TA>
__global__ void __launch_bounds__(128)
gated_norm_kernel(const float* __restrict__ o, const float* __restrict__ w, int w_len, const TA* __restrict__ gate,
                  long ldg, float eps, TA* __restrict__ out, long pairs, int groups, int n) {
    const long pair = (long)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (pair >= pairs) return;
    const long t = pair / groups;
    const int g = (int)(pair - t * groups);
    const float* row = o + (t * groups + g) * n;
    float ss = 0.f;
    for (int i = lane; i < n; i += 32) ss = fmaf(row[i], row[i], ss);
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)n + eps);
    for (int i = lane; i < n; i += 32) {
        const int c = g * n + i;
        const float gv = to_float(gate[t * ldg + c]);
        out[(t * groups + g) * n + i] = from_float<TA>(row[i] * inv * w[c % w_len] * (1.f / (1.f + expf(-gv))));
    }
}

template <typename TA, bool DELTA>
int launch_scan(const void* q, const void* k, const void* v, long ld, int group, const float* a, const void* b,
                long ldb, const float* a_log, const float* dt_bias, const float* decay, float* state, float* out,
                const int* seg_q_start, const int* seg_slot, int segments, int H, int D, int V, int silu_inputs,
                cudaStream_t stream) {
    const int dpt = D <= 32 ? 32 : D <= 64 ? 64 : 128;
    const int DS = (D + dpt - 1) / dpt;
    const dim3 grid((V + 31) / 32, H, segments), block(32, DS);
    const size_t smem = sizeof(float) * ((size_t)SCAN_TOKENS * D * (DELTA ? 3 : 2) + SCAN_TOKENS * 33 + DS * 32);
#define MRUN_SCAN(DPT)                                                                                        \
    scan_kernel<TA, DPT, DELTA><<<grid, block, smem, stream>>>((const TA*)q, (const TA*)k, (const TA*)v, ld,  \
        group, a, (const TA*)b, ldb, a_log, dt_bias, decay, state, out, seg_q_start, seg_slot, H, D, V, silu_inputs)
    if (dpt == 32) MRUN_SCAN(32);
    else if (dpt == 64) MRUN_SCAN(64);
    else MRUN_SCAN(128);
#undef MRUN_SCAN
    return 0;
}

}  // namespace

// x: row t at x + t * ldx, C channels; w: float32 [C, taps]; state: [slots, taps - 1, C] in the
// activation dtype; out: row t at out + t * ldo.  seg_q_start: int32 [segments + 1].
MRUN_API int mrun_causal_conv(const void* x, long ldx, const float* w, void* state, void* out, long ldo, int act_dtype,
                              const int* seg_q_start, const int* seg_slot, int segments, int max_q_len, int C,
                              int taps, int residual, int silu, cudaStream_t stream) {
    MRUN_REQUIRE(C > 0 && segments >= 0 && max_q_len >= 0, "causal_conv: bad sizes");
    MRUN_REQUIRE(taps >= 2 && taps <= MAX_TAPS, "causal_conv: %d taps, the kernel takes 2 to %d", taps, MAX_TAPS);
    MRUN_REQUIRE(ldx >= C && ldo >= C, "causal_conv: a row stride below the %d channels", C);
    MRUN_REQUIRE(segments <= 65535, "causal_conv: %d segments exceed 65535", segments);
    if (segments == 0 || max_q_len == 0) return 0;
    const int tiles = (max_q_len + CONV_TILE - 1) / CONV_TILE;
    MRUN_REQUIRE(tiles <= 65535, "causal_conv: a segment of %d tokens is too long", max_q_len);
    const dim3 grid((C + 127) / 128, tiles, segments);
    if (act_dtype == MRUN_F32)
        causal_conv_kernel<float><<<grid, 128, 0, stream>>>((const float*)x, ldx, w, (float*)state, (float*)out, ldo,
                                                             seg_q_start, seg_slot, C, taps, residual, silu);
    else if (act_dtype == MRUN_BF16)
        causal_conv_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(
            (const __nv_bfloat16*)x, ldx, w, (__nv_bfloat16*)state, (__nv_bfloat16*)out, ldo, seg_q_start, seg_slot, C,
            taps, residual, silu);
    else
        return mrun_set_error("causal_conv: unknown dtype code %d", act_dtype);
    MRUN_CHECK_LAUNCH("causal_conv");
    return 0;
}

// q, k: row t at + t * ld, [H / group heads, D]; v: [H, V] likewise.  state: float32 [slots, H, D, V];
// out: float32 [tokens, H * V].  decay: float32 [H].
MRUN_API int mrun_decay_scan(const void* q, const void* k, const void* v, long ld, int act_dtype, const float* decay,
                             float* state, float* out, const int* seg_q_start, const int* seg_slot, int segments,
                             int H, int D, int V, int silu_inputs, cudaStream_t stream) {
    MRUN_REQUIRE(H > 0 && D > 0 && V > 0 && segments >= 0, "decay_scan: bad sizes");
    MRUN_REQUIRE(D <= 256, "decay_scan: key size %d exceeds the supported 256", D);
    MRUN_REQUIRE(H <= 65535 && segments <= 65535, "decay_scan: %d heads or %d segments exceed 65535", H, segments);
    if (segments == 0) return 0;
    if (act_dtype == MRUN_F32)
        launch_scan<float, false>(q, k, v, ld, 1, nullptr, nullptr, 0, nullptr, nullptr, decay, state, out, seg_q_start,
                                  seg_slot, segments, H, D, V, silu_inputs, stream);
    else if (act_dtype == MRUN_BF16)
        launch_scan<__nv_bfloat16, false>(q, k, v, ld, 1, nullptr, nullptr, 0, nullptr, nullptr, decay, state, out,
                                          seg_q_start, seg_slot, segments, H, D, V, silu_inputs, stream);
    else
        return mrun_set_error("decay_scan: unknown dtype code %d", act_dtype);
    MRUN_CHECK_LAUNCH("decay_scan");
    return 0;
}

// q, k: [H / group heads, D] a row (stride ld); v: [H, V] (stride ld); a: float32 [tokens, H * D];
// b: row t at b + t * ldb, [H]; a_log: float32 [H]; dt_bias: float32 [H * D].
MRUN_API int mrun_delta_scan(const void* q, const void* k, const void* v, long ld, int act_dtype, int group,
                             const float* a, const void* b, long ldb, const float* a_log, const float* dt_bias,
                             float* state, float* out, const int* seg_q_start, const int* seg_slot, int segments,
                             int H, int D, int V, cudaStream_t stream) {
    MRUN_REQUIRE(H > 0 && D > 0 && V > 0 && segments >= 0 && group > 0 && H % group == 0, "delta_scan: bad sizes");
    MRUN_REQUIRE(D <= 256, "delta_scan: key size %d exceeds the supported 256", D);
    MRUN_REQUIRE(H <= 65535 && segments <= 65535, "delta_scan: %d heads or %d segments exceed 65535", H, segments);
    if (segments == 0) return 0;
    if (act_dtype == MRUN_F32)
        launch_scan<float, true>(q, k, v, ld, group, a, b, ldb, a_log, dt_bias, nullptr, state, out, seg_q_start,
                                 seg_slot, segments, H, D, V, 0, stream);
    else if (act_dtype == MRUN_BF16)
        launch_scan<__nv_bfloat16, true>(q, k, v, ld, group, a, b, ldb, a_log, dt_bias, nullptr, state, out,
                                         seg_q_start, seg_slot, segments, H, D, V, 0, stream);
    else
        return mrun_set_error("delta_scan: unknown dtype code %d", act_dtype);
    MRUN_CHECK_LAUNCH("delta_scan");
    return 0;
}

// o: float32 [tokens, groups * n]; w: float32 [w_len], element c of a row takes w[c % w_len];
// gate: row t at gate + t * ldg; out: dense [tokens, groups * n].
MRUN_API int mrun_gated_norm(const float* o, const float* w, int w_len, const void* gate, long ldg, int act_dtype,
                             float eps, void* out, int tokens, int groups, int n, cudaStream_t stream) {
    MRUN_REQUIRE(tokens >= 0 && groups > 0 && n > 0 && w_len > 0, "gated_norm: bad sizes");
    MRUN_REQUIRE(ldg >= (long)groups * n, "gated_norm: the gate's row stride %ld is below the row", ldg);
    if (tokens == 0) return 0;
    const long pairs = (long)tokens * groups;
    const unsigned blocks = (unsigned)((pairs + 3) / 4);
    if (act_dtype == MRUN_F32)
        gated_norm_kernel<float><<<blocks, 128, 0, stream>>>(o, w, w_len, (const float*)gate, ldg, eps, (float*)out,
                                                              pairs, groups, n);
    else if (act_dtype == MRUN_BF16)
        gated_norm_kernel<__nv_bfloat16><<<blocks, 128, 0, stream>>>(o, w, w_len, (const __nv_bfloat16*)gate, ldg, eps,
                                                                      (__nv_bfloat16*)out, pairs, groups, n);
    else
        return mrun_set_error("gated_norm: unknown dtype code %d", act_dtype);
    MRUN_CHECK_LAUNCH("gated_norm");
    return 0;
}
