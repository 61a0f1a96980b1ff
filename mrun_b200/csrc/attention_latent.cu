// Paged attention over wide latent rows on the tensor cores (mma.sync), bfloat16: every query head
// of a token meets the same cache rows, a row is the key (all `width` features) and, in its
// first `value_cols` features, the value.  For rows wider than the 256 features the per-head-size
// kernels are built for (a latent of 512 and a rotated part of 64, say).
//
// One block of four warps takes one token and up to 16 of its heads (the 16 rows of the
// m16n8k16 products) and walks over the token's keys in tiles of 32, copied with cp.async (into a
// ring of two, or into a single stage where the launch has blocks enough to overlap one another):
//   S = Q K^T   warp w takes keys 8w .. 8w+7 of the tile and all of the row's features; scores go
//               to shared memory, scaled, keys after the token's position masked
//   softmax     eight threads a row: running maximum and total in 32-bit, P as bfloat16
//   O += P V    warp w keeps a quarter of the value columns in registers (up to 128 columns,
//               so value_cols <= 512) and reads V from the same tile of shared memory
// Keys outside the token's range are copied as zeros, so a masked key adds exactly nothing.  A
// step of few tokens deals every token's tiles to several blocks (grid.z), which leave their
// unnormalised sums in scratch for a merge kernel that adds them in a fixed order.
#include "attention_paging.cuh"
#include "common.cuh"

using namespace mrun;

namespace {

using bf16 = __nv_bfloat16;
constexpr int TILE_KEYS = 32, ROWS = 16, THREADS = 128, MAX_TILES_A_WARP = 16;
constexpr int MIN_RUN = 8;          // the fewest key tiles a block of a split launch takes
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ unsigned smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async_16(void* dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes become zero
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// grid: (tokens, head groups of 16, splits).
template <int STAGES>
__global__ void __launch_bounds__(THREADS)
latent_wide_kernel(const bf16* __restrict__ q, long q_stride, bf16* __restrict__ out, const bf16* __restrict__ cache,
                   const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ token_slot,
                   const int* __restrict__ positions, int heads, int width, int value_cols, int page_size,
                   int page_shift, float scale, int splits, float* __restrict__ part_o, float* __restrict__ part_ml) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int ld = width + 8;                                   // row stride in elements: an odd number of 16-byte chunks
    bf16* q_tile = reinterpret_cast<bf16*>(smem_raw);           // [ROWS][ld]
    bf16* k_ring = q_tile + ROWS * ld;                          // [STAGES][TILE_KEYS][ld]
    float* scores = reinterpret_cast<float*>(k_ring + STAGES * TILE_KEYS * ld); // [ROWS][TILE_KEYS + 1]
    bf16* probs = reinterpret_cast<bf16*>(scores + ROWS * (TILE_KEYS + 1));     // [ROWS][TILE_KEYS + 8]
    float* row_max = reinterpret_cast<float*>(probs + ROWS * (TILE_KEYS + 8));  // [ROWS]
    float* row_sum = row_max + ROWS;                                            // [ROWS]
    float* row_corr = row_sum + ROWS;                                           // [ROWS]

    const int t = blockIdx.x, head0 = blockIdx.y * ROWS;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
    const int pos = positions[t];
    const int rows_here = min(ROWS, heads - head0);
    if (pos < 0) {                                              // a padding row of the step
        for (int i = tid; i < rows_here * width; i += THREADS)
            out[((size_t)t * heads + head0) * width + i] = __float2bfloat16_rn(0.f);
        return;
    }
    const int chunks = width >> 3;
    Paging pg{block_tables + (size_t)token_slot[t] * max_blocks, 1, 0, page_size, page_shift};

    // a warp takes every fourth key of the tile: one look at the block table a key, then the
    // row's 16-byte chunks lane by lane
    auto load_tile = [&](int tile, int stage) {
        bf16* dst = k_ring + (size_t)stage * TILE_KEYS * ld;
        for (int key_in = warp; key_in < TILE_KEYS; key_in += THREADS / 32) {
            const int key = tile * TILE_KEYS + key_in;
            bool valid = key <= pos;
            // cache_row's template argument is a compile-time head size; the width is a run-time
            // value here, so the row number is asked for with size 1 and scaled
            const long row = cache_row<1>(pg, key, valid);
            const bf16* src = cache + (valid ? row * width : 0);
            for (int c = lane; c < chunks; c += 32) cp_async_16(dst + key_in * ld + c * 8, src + c * 8, valid);
        }
    };

    // with `splits` > 1 the token's tiles are dealt to gridDim.z blocks in equal runs; a block
    // leaves its unnormalised sums, maxima and totals in the scratch arrays for the merge kernel
    const int all_tiles = pos / TILE_KEYS + 1;
    // at least MIN_RUN tiles a block: a captured step is launched with the splits of its longest
    // possible context, and a shorter token leaves the later blocks without tiles (an empty piece)
    const int run = max((all_tiles + splits - 1) / splits, splits > 1 ? MIN_RUN : 1);
    const int tile_begin = blockIdx.z * run;
    const int tiles = min(all_tiles, tile_begin + run);
    if (STAGES > 1 && tile_begin < tiles) load_tile(tile_begin, 0);
    cp_async_commit();
    // the token's queries: rows beyond the heads of this group are zeros
    for (int i = tid; i < ROWS * chunks; i += THREADS) {
        const int r = i / chunks, c = i - r * chunks;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < rows_here) v = *reinterpret_cast<const uint4*>(q + (size_t)t * q_stride + (size_t)(head0 + r) * width + c * 8);
        *reinterpret_cast<uint4*>(q_tile + r * ld + c * 8) = v;
    }
    if (tid < ROWS) { row_max[tid] = -INFINITY; row_sum[tid] = 0.f; }

    // the warp's value columns: n-tiles of 8, an even count a warp
    const int value_tiles = (value_cols + 7) >> 3;
    int tiles_a_warp = (value_tiles + 3) >> 2;
    tiles_a_warp += tiles_a_warp & 1;
    const int first_tile = warp * tiles_a_warp;
    const int last_tile = min(first_tile + tiles_a_warp, chunks);      // columns past the row do not exist
    float acc[MAX_TILES_A_WARP][4];
#pragma unroll
    for (int j = 0; j < MAX_TILES_A_WARP; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

    const float scale2 = scale * LOG2E;
    for (int tile = tile_begin; tile < tiles; ++tile) {
        const int stage = STAGES > 1 ? (tile - tile_begin) & 1 : 0;
        if constexpr (STAGES > 1) {
            if (tile + 1 < tiles) load_tile(tile + 1, stage ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {                                               // one stage: other blocks of the multiprocessor compute meanwhile
            load_tile(tile, 0);
            cp_async_commit();
            cp_async_wait<0>();
        }
        __syncthreads();
        const bf16* k_tile = k_ring + (size_t)stage * TILE_KEYS * ld;

        // ---- S = Q K^T: this warp's eight keys
        {
            // four sums side by side (one a 16-feature step of each 64), so that a product does not
            // wait for the one before it; they are added in a fixed order at the end
            float s[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f}, s2[4] = {0.f, 0.f, 0.f, 0.f},
                  s3[4] = {0.f, 0.f, 0.f, 0.f};
            const bf16* a_ptr = q_tile + (lane & 15) * ld + (lane >> 4) * 8;
            const bf16* b_ptr = k_tile + (warp * 8 + (lane & 7)) * ld + (lane >> 3) * 8;
            int k0 = 0;
            for (; k0 + 64 <= width; k0 += 64) {
                unsigned a0[4], a1[4], a2[4], a3[4], b0[4], b1[4];
                ldmatrix_x4(a0, a_ptr + k0);
                ldmatrix_x4(a1, a_ptr + k0 + 16);
                ldmatrix_x4(a2, a_ptr + k0 + 32);
                ldmatrix_x4(a3, a_ptr + k0 + 48);
                ldmatrix_x4(b0, b_ptr + k0);
                ldmatrix_x4(b1, b_ptr + k0 + 32);
                mma_bf16(s, a0, b0[0], b0[1]);
                mma_bf16(s1, a1, b0[2], b0[3]);
                mma_bf16(s2, a2, b1[0], b1[1]);
                mma_bf16(s3, a3, b1[2], b1[3]);
            }
            for (; k0 < width; k0 += 16) {                      // the last 16, 32 or 48 features
                unsigned a0[4], b[4];
                ldmatrix_x4(a0, a_ptr + k0);
                // lanes 16..31 would address features past the step: they repeat the first half
                ldmatrix_x4(b, k_tile + (warp * 8 + (lane & 7)) * ld + ((lane >> 3) & 1) * 8 + k0);
                mma_bf16(s, a0, b[0], b[1]);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) s[i] = (s[i] + s1[i]) + (s2[i] + s3[i]);
            const int key0 = tile * TILE_KEYS + warp * 8 + 2 * tq;
            float* s_row = scores + g * (TILE_KEYS + 1) + warp * 8 + 2 * tq;
            s_row[0] = key0 <= pos ? s[0] * scale2 : -INFINITY;
            s_row[1] = key0 + 1 <= pos ? s[1] * scale2 : -INFINITY;
            s_row += 8 * (TILE_KEYS + 1);
            s_row[0] = key0 <= pos ? s[2] * scale2 : -INFINITY;
            s_row[1] = key0 + 1 <= pos ? s[3] * scale2 : -INFINITY;
        }
        __syncthreads();

        // ---- softmax: eight threads a row, four keys each (scores are in units of log2 e)
        {
            const int r = tid >> 3, part = tid & 7;
            float v[4];
            float m = -INFINITY;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                v[i] = scores[r * (TILE_KEYS + 1) + part * 4 + i];
                m = fmaxf(m, v[i]);
            }
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            const float m_old = row_max[r];
            const float m_new = fmaxf(m_old, m);                // finite: the tile's first key is visible
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float p = exp2f(v[i] - m_new);
                const bf16 pb = __float2bfloat16_rn(p);
                probs[r * (TILE_KEYS + 8) + part * 4 + i] = pb;
                sum += __bfloat162float(pb);                     // the total of what the product sees
            }
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            __syncwarp();
            if (part == 0) {
                const float corr = exp2f(m_old - m_new);        // 0 at the first tile
                row_corr[r] = corr;
                row_sum[r] = row_sum[r] * corr + sum;
                row_max[r] = m_new;
            }
        }
        __syncthreads();

        // ---- O += P V: this warp's value columns
        {
            const float c_lo = row_corr[g], c_hi = row_corr[g + 8];
            unsigned p0[4], p1[4];
            ldmatrix_x4(p0, probs + (lane & 15) * (TILE_KEYS + 8) + (lane >> 4) * 8);
            ldmatrix_x4(p1, probs + (lane & 15) * (TILE_KEYS + 8) + 16 + (lane >> 4) * 8);
            // lanes 0..7: keys 0..7 of n-tile j, 8..15: keys 8..15, 16..23 and 24..31: the same of n-tile j + 1
            const bf16* v_ptr = k_tile + ((lane & 7) + ((lane >> 3) & 1) * 8) * ld + (lane >> 4) * 8;
#pragma unroll
            for (int j = 0; j < MAX_TILES_A_WARP; j += 2) {
                const int n_tile = first_tile + j;
                if (n_tile < last_tile) {
                    acc[j][0] *= c_lo; acc[j][1] *= c_lo; acc[j][2] *= c_hi; acc[j][3] *= c_hi;
                    acc[j + 1][0] *= c_lo; acc[j + 1][1] *= c_lo; acc[j + 1][2] *= c_hi; acc[j + 1][3] *= c_hi;
                    // an odd number of n-tiles in the row: the second tile of the last pair repeats the first
                    const int second = n_tile + 1 < chunks ? 8 : 0;
                    unsigned b[4];
                    ldmatrix_x4_trans(b, v_ptr + n_tile * 8 + (lane >> 4) * (second - 8));
                    mma_bf16(acc[j], p0, b[0], b[1]);
                    mma_bf16(acc[j + 1], p0, b[2], b[3]);
                    ldmatrix_x4_trans(b, v_ptr + 16 * ld + n_tile * 8 + (lane >> 4) * (second - 8));
                    mma_bf16(acc[j], p1, b[0], b[1]);
                    mma_bf16(acc[j + 1], p1, b[2], b[3]);
                }
            }
        }
        __syncthreads();                                        // the tile, the scores and P are free again
    }

    if (splits > 1) {
        __syncthreads();                                        // a block without tiles still owes its (empty) piece
        const size_t piece = ((size_t)t * gridDim.y + blockIdx.y) * splits + blockIdx.z;
        const int cols = 4 * tiles_a_warp * 8;                  // columns a piece holds (those of all four warps)
        float* o = part_o + piece * ROWS * cols;
#pragma unroll
        for (int j = 0; j < MAX_TILES_A_WARP; ++j) {
            const int n_tile = first_tile + j;
            if (j < tiles_a_warp) {
                const int col = n_tile * 8 + 2 * tq;
                *reinterpret_cast<float2*>(o + g * cols + col) = make_float2(acc[j][0], acc[j][1]);
                *reinterpret_cast<float2*>(o + (g + 8) * cols + col) = make_float2(acc[j][2], acc[j][3]);
            }
        }
        if (tid < ROWS) {
            part_ml[(piece * ROWS + tid) * 2] = row_max[tid];
            part_ml[(piece * ROWS + tid) * 2 + 1] = row_sum[tid];
        }
        return;
    }
    // ---- out = O / l
    const float inv_lo = 1.f / row_sum[g], inv_hi = 1.f / row_sum[g + 8];
#pragma unroll
    for (int j = 0; j < MAX_TILES_A_WARP; ++j) {
        const int n_tile = first_tile + j;
        if (n_tile < last_tile) {
            const int col = n_tile * 8 + 2 * tq;
            if (g < rows_here)
                *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)t * heads + head0 + g) * width + col) =
                    __floats2bfloat162_rn(acc[j][0] * inv_lo, acc[j][1] * inv_lo);
            if (g + 8 < rows_here)
                *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)t * heads + head0 + g + 8) * width + col) =
                    __floats2bfloat162_rn(acc[j][2] * inv_hi, acc[j][3] * inv_hi);
        }
    }
}

// The pieces of a (token, head) added up: out = sum_s O_s 2^(m_s - M) / sum_s l_s 2^(m_s - M), in the
// order of s.  grid: (tokens, heads); a block's threads share the row's weights and walk its columns.
// A piece without tiles has m = -inf and counts nothing.
constexpr int MAX_SPLITS = 64;

__global__ void __launch_bounds__(128)
latent_wide_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                         bf16* __restrict__ out, const int* __restrict__ positions, int heads, int width,
                         int cols, int splits) {
    __shared__ float weight[MAX_SPLITS];
    __shared__ float inv_total;
    const int t = blockIdx.x, head = blockIdx.y;
    if (positions[t] < 0) return;                               // the attention kernel wrote zeros
    const int groups = (heads + ROWS - 1) / ROWS;
    const size_t first = ((size_t)t * groups + head / ROWS) * splits;
    const int r = head % ROWS;
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        float m = -INFINITY;
        for (int s = lane; s < splits; s += 32) m = fmaxf(m, part_ml[((first + s) * ROWS + r) * 2]);
        m = warp_max(m);
        float total = 0.f;
        for (int s0 = 0; s0 < splits; s0 += 32) {               // the totals are added in the order of s
            const int s = s0 + lane;
            float w = 0.f, l = 0.f;
            if (s < splits) {
                const float ms = part_ml[((first + s) * ROWS + r) * 2];
                w = ms == -INFINITY ? 0.f : exp2f(ms - m);
                l = part_ml[((first + s) * ROWS + r) * 2 + 1] * w;
                weight[s] = w;
            }
            for (int i = 0; i < 32; ++i) total += __shfl_sync(0xffffffffu, l, i);
        }
        if (lane == 0) inv_total = 1.f / total;
    }
    __syncthreads();
    const int out_cols = min(cols, width);
    for (int c = threadIdx.x; c < out_cols; c += blockDim.x) {
        float value = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float w = weight[s];
            if (w != 0.f) value += part_o[((first + s) * ROWS + r) * (size_t)cols + c] * w;
        }
        out[((size_t)t * heads + head) * width + c] = __float2bfloat16_rn(value * inv_total);
    }
}

size_t latent_wide_smem(int width, int stages = 2) {
    const size_t ld = width + 8;
    return (ROWS + stages * TILE_KEYS) * ld * sizeof(bf16) + ROWS * (TILE_KEYS + 1) * sizeof(float) +
           ROWS * (TILE_KEYS + 8) * sizeof(bf16) + 3 * ROWS * sizeof(float);
}

}  // namespace

// Whether mrun_latent_attention_wide takes rows of `width` features with `value_cols` value columns.
MRUN_API int mrun_latent_attention_wide_ok(int width, int value_cols) {
    return width % 16 == 0 && width >= 32 && value_cols > 0 && value_cols <= width &&
           value_cols <= 4 * MAX_TILES_A_WARP * 8 && latent_wide_smem(width) <= 200 * 1024;
}

// Columns a piece of a split launch holds for each of its 16 rows.
MRUN_API int mrun_latent_attention_wide_piece_cols(int value_cols) {
    int tiles_a_warp = ((value_cols + 7) / 8 + 3) / 4;
    tiles_a_warp += tiles_a_warp & 1;
    return 4 * tiles_a_warp * 8;
}

// q: row t starts at q + t * q_stride, heads contiguous [heads, width].  out: dense [tokens, heads * width];
// the first value_cols features of every head are written (rounded up to whole pairs of 8).
// cache: [pages, 1, page_size, width].  positions[t] < 0 = padding.  splits > 1 (few tokens, long
// contexts): every token's keys are dealt to that many blocks; part_o holds
// [tokens, head groups, splits, 16, piece_cols] floats and part_ml [.., 16, 2].
MRUN_API int mrun_latent_attention_wide(const void* q, long q_stride, void* out, const void* cache,
                                        const int* block_tables, int max_blocks, const int* token_slot,
                                        const int* positions, int tokens, int heads, int width, int value_cols,
                                        int page_size, long cache_rows, float scale, int splits, float* part_o,
                                        float* part_ml, cudaStream_t stream) {
    MRUN_REQUIRE(splits >= 1 && splits <= MAX_SPLITS && heads <= 65535 && (splits == 1 || (part_o != nullptr && part_ml != nullptr)),
                 "latent_attention_wide: splits=%d needs scratch for the pieces", splits);
    MRUN_REQUIRE(tokens >= 0 && heads > 0 && page_size > 0 && max_blocks > 0, "latent_attention_wide: bad sizes");
    MRUN_REQUIRE(mrun_latent_attention_wide_ok(width, value_cols),
                 "latent_attention_wide: rows of %d features with %d value columns are not supported", width, value_cols);
    MRUN_REQUIRE(cache_rows < (1L << 31) / 1, "latent_attention_wide: the cache has %ld rows, the limit is 2^31", cache_rows);
    MRUN_REQUIRE((((uintptr_t)q | (uintptr_t)out | (uintptr_t)cache) & 15) == 0 && q_stride % 8 == 0,
                 "latent_attention_wide: q, out and the cache must be 16-byte aligned");
    MRUN_REQUIRE((heads + ROWS - 1) / ROWS <= 65535, "latent_attention_wide: heads=%d", heads);
    if (tokens == 0) return 0;
    // A launch that fills the device three times over runs with one stage of keys (60 KB of shared
    // memory at 576 features: three blocks a multiprocessor, and while one waits for its tile the
    // others compute; measured on B200 at 2,048 tokens of 16 heads: 0.80 against 0.98 ms); a
    // smaller launch keeps the ring of two, where a block's own next tile is all there is to overlap.
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms < 1)
            sms = 148;
    }
    const long blocks = (long)tokens * ((heads + ROWS - 1) / ROWS) * splits;
    const int stages = blocks >= 3L * sms ? 1 : 2;
    const size_t smem = latent_wide_smem(width, stages);
    auto kernel = stages == 1 ? latent_wide_kernel<1> : latent_wide_kernel<2>;
    MRUN_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                    "latent_attention_wide");
    const dim3 grid(tokens, (heads + ROWS - 1) / ROWS, splits);
    kernel<<<grid, THREADS, smem, stream>>>((const bf16*)q, q_stride, (bf16*)out, (const bf16*)cache,
                                                        block_tables, max_blocks, token_slot, positions, heads, width,
                                                        value_cols, page_size, page_shift_of(page_size), scale, splits,
                                                        part_o, part_ml);
    MRUN_CHECK_LAUNCH("latent_attention_wide");
    if (splits > 1) {
        latent_wide_merge_kernel<<<dim3(tokens, heads), 128, 0, stream>>>(
            part_o, part_ml, (bf16*)out, positions, heads, width, mrun_latent_attention_wide_piece_cols(value_cols), splits);
        MRUN_CHECK_LAUNCH("latent_attention_wide (merge)");
    }
    return 0;
}
