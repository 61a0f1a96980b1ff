"""Balivik on the GPU against the plain implementation (``plain_balivik``): every kernel and every
mixer alone (whole requests, token by token, portions down to one and two tokens, unequal requests
side by side, state slots and pages given back and used again), then whole models replayed through
``bin/trace_run`` cut in every way, then greedy generation through ``Engine.generate`` and the
command line."""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import plain_balivik as plain
from tiny_balivik import BTINY, load_folder, make_folder, tokens_of
from trace_tools import TraceBuilder, TraceRunner, cut_decode_tail, cut_mixed, cut_portions, cut_whole

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


def runtime(dtype, page_size=8):
    from mrun_b200.parts import Precision, Runtime
    return Runtime(torch.device(DEV), Precision.of(dtype), page_size)


def tolerance(dtype):
    return 3e-5 if dtype == "float32" else 3e-2


def close(got, want, dtype, what="", bound=None):
    got, want = got.detach().to("cpu", F64), want.to(F64)
    error = float((got - want).abs().max() / want.abs().max())
    assert error <= (bound or tolerance(dtype)), f"{what}: relative error {error:.3e}"


class Steps:
    """A cache manager for one schedule entry's need and step contexts for several requests."""

    def __init__(self, need, rt, pages=96, slots=3):
        from mrun_b200.cache import CacheManager
        from mrun_b200.engine.batch import HostStaging
        self.manager = CacheManager([need], [None], rt.page_size, pages, slots, device=rt.device, dtype=rt.precision.act)
        self.staging = HostStaging(rt.device)
        self.cache = self.manager.entries[0]
        self.requests = {}

    def run(self, entries, fn):
        """entries: [(request id, tokens)]; ``fn(ctx, places)`` runs the step, places = [(id, first
        position, first row, tokens)]; the step is committed after it."""
        from mrun_b200.engine.batch import StepEntry, build_context
        for rid, _ in entries:
            if rid not in self.requests:
                self.requests[rid] = self.manager.admit(rid)
        items = [(self.requests[rid], n) for rid, n in entries]
        starts = [r.length for r, _ in items]
        plan = self.manager.plan_append(items)
        ctx = build_context([StepEntry(r, [0] * n) for r, n in items], self.manager, self.staging)
        places = [(rid, start, seg.q_start, n) for (rid, n), start, seg in zip(entries, starts, ctx.segments)]
        out = fn(ctx, places)
        self.manager.commit(plan)
        return out

    def release(self, rid):
        self.manager.release(self.requests.pop(rid))


def schedules(lengths):
    """Ways of feeding the same requests: (label, steps, slots); a step is [(id, tokens)] and an id
    ending a step with 'end' is released after it."""
    ids = list(lengths)
    out = [("whole", [[(r, lengths[r])] for r in ids], 2)]
    steps = []
    for r in ids:                               # a prefix, then token by token
        head = max(1, lengths[r] - 40)
        steps += [[(r, head)]] + [[(r, 1)] for _ in range(lengths[r] - head)]
    out.append(("token by token", steps, 2))
    sizes = [2, 7, 1, 3, 16, 5, 2, 33, 9, 64, 4, 1]
    steps, k = [], 0
    for r in ids:                               # portions of changing size
        at = 0
        while at < lengths[r]:
            n = min(sizes[k % len(sizes)], lengths[r] - at)
            k += 1
            steps.append([(r, n)])
            at += n
    out.append(("portions", steps, 2))
    # unequal requests side by side, three at a time: portions of some beside single tokens of others
    rng = np.random.default_rng(5)
    waiting, running, steps = list(ids), {}, []
    while waiting or running:
        while waiting and len(running) < 3:
            running[waiting.pop(0)] = 0
        step = []
        for r in list(running):
            left = lengths[r] - running[r]
            if rng.random() < 0.25 and len(running) > 1:
                continue
            n = 1 if left <= 6 else min(int(rng.choice(sizes)), left - 6)
            step.append((r, n))
            running[r] += n
            if running[r] == lengths[r]:
                del running[r]
        if step:
            steps.append(step)
    out.append(("side by side", steps, 3))
    return out


def check_mixer(part, hidden, dtype, lengths, plain_fn, need=None, rt=None, bound=None, inputs=None):
    """Runs ``part`` over random inputs fed by every schedule and compares each request's rows with
    ``plain_fn(x)`` of the whole request; in 32-bit all schedules must give the same bits."""
    gen = torch.Generator().manual_seed(11)
    act = rt.precision.act
    x = inputs or {r: torch.randn(n, hidden, generator=gen) for r, n in lengths.items()}
    x = {r: v.to(act).to(torch.float32) for r, v in x.items()}           # what the part really sees
    want = {r: plain_fn(v.to(F64)) for r, v in x.items()}
    scale = max(float(w.abs().max()) for w in want.values())
    first = {}
    for label, steps, slots in schedules(lengths):
        book = Steps(need if need is not None else part.cache_need(), rt, slots=slots)
        fed = {r: 0 for r in lengths}

        def run(ctx, places):
            rows = torch.cat([x[rid][start:start + n] for rid, start, _, n in places]).to(DEV, act)
            return part.forward(rows, ctx, book.cache).float().cpu()

        for step in steps:
            out = book.run(step, run)
            at = 0
            for rid, n in step:
                got, start = out[at:at + n], fed[rid]
                error = float((got.to(F64) - want[rid][start:start + n]).abs().max()) / scale
                assert error <= (bound or tolerance(dtype)), f"{label}: request {rid}, tokens {start}..{start + n}: {error:.3e}"
                if dtype == "float32":
                    for i in range(n):
                        seen = first.setdefault((rid, start + i), got[i])
                        assert torch.equal(seen, got[i]), f"{label}: request {rid}, position {start + i} differs in bits"
                at += n
                fed[rid] += n
                if fed[rid] == lengths[rid]:
                    book.release(rid)                              # its slot and pages are used again
        book.manager.check_invariants()


# ------------------------------------------------------------------ kernels alone

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_streams_step_kernel(dtype):
    from mrun_b200.kernels import ops
    act = torch.float32 if dtype == "float32" else torch.bfloat16
    gen = torch.Generator().manual_seed(2)
    for count, width in ((1, 100), (2, 64), (3, 257), (8, 1000)):
        streams = torch.randn(7, count, width, generator=gen).to(DEV)
        y = torch.randn(7, width, generator=gen).to(DEV)
        mix, out_c, in_c = (torch.randn(*s, generator=gen).to(DEV) for s in ((count, count), (count,), (count,)))
        norm_w = (1 + 0.2 * torch.randn(width, generator=gen)).to(DEV)
        old = streams.cpu().double()
        new = torch.einsum("sr,tsw->trw", mix.cpu().double(), old) + out_c.cpu().double()[None, :, None] * y.cpu().double()[:, None, :]
        u = torch.einsum("s,tsw->tw", in_c.cpu().double(), new)
        rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
        flat = streams.reshape(7, count * width).clone()
        pending = ops.PendingStreams(y, mix, out_c)
        total = ops.streams_step(flat, pending, None, None, 0.0, torch.float32, count, rows=rows, want_sum=True)
        assert torch.equal(flat, streams.reshape(7, -1))                   # with rows the streams stay
        close(total, new.sum(1)[[6, 0, 3]], "float32", "sum of the streams at rows")
        h = ops.streams_step(flat, pending, in_c, norm_w, 1e-5, act, count)
        close(flat.reshape(7, count, width), new, "float32", "streams after the write")
        close(h, plain.rms_norm(u, norm_w.cpu().double(), 1e-5), dtype, "normed read")
        # no pending write: the streams stay; plain residual sum with one stream and no coefficients
        before = flat.clone()
        h = ops.streams_step(flat, None, in_c, norm_w, 1e-5, act, count)
        assert torch.equal(flat, before)
        close(h, plain.rms_norm(u, norm_w.cpu().double(), 1e-5), dtype, "read without a write")
    one = torch.randn(5, 96, generator=gen).to(DEV)
    y = torch.randn(5, 96, generator=gen).to(DEV)
    w = torch.ones(96, device=DEV)
    h = ops.streams_step(one, ops.PendingStreams(y, None, None), None, w, 1e-6, act, 1)
    close(h, plain.rms_norm(one.cpu().double(), 1.0, 1e-6), dtype, "x += y, then the norm")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("taps, channels, residual", [(2, 100, True), (4, 64, True), (3, 200, False), (8, 33, False),
                                                      (1, 40, True), (1, 9, False)])
def test_causal_conv_with_state(dtype, taps, channels, residual):
    """Requests fed in portions down to one token, side by side, with slots used again: every
    output equals the convolution over the whole request, zeros before its start."""
    from mrun_b200.cache.needs import FixedState
    from mrun_b200.kernels import ops
    rt = runtime(dtype)
    act = rt.precision.act
    gen = torch.Generator().manual_seed(taps)
    weight = torch.randn(channels, taps, generator=gen)
    lengths = {"a": 70, "b": 3, "c": 131, "d": 1, "e": 66}
    x = {r: torch.randn(n, channels, generator=gen).to(act).float() for r, n in lengths.items()}
    want = {}
    for r, v in x.items():
        y = plain.causal_conv(v.double(), weight.double())
        want[r] = v.double() + y if residual else plain.silu(y)
    for label, steps, slots in schedules(lengths):
        book = Steps(FixedState((taps - 1, channels), rt.precision.name, name="conv"), rt, slots=slots)
        fed = {r: 0 for r in lengths}
        for step in steps:
            def run(ctx, places):
                rows = torch.cat([x[rid][start:start + n] for rid, start, _, n in places]).to(DEV, act)
                wide = torch.zeros(rows.shape[0], channels + 24, dtype=act, device=DEV)      # a column slice of a wider matrix
                wide[:, 8:8 + channels] = rows
                return ops.causal_conv(wide[:, 8:8 + channels], weight.to(DEV), book.cache.states["conv"], ctx,
                                       residual=residual, silu=not residual).float().cpu()
            out = book.run(step, run)
            at = 0
            for rid, n in step:
                close(out[at:at + n], want[rid][fed[rid]:fed[rid] + n], dtype, f"{label}: {rid} from {fed[rid]}",
                      bound=2e-6 if dtype == "float32" else 2e-2)
                at += n
                fed[rid] += n
                if fed[rid] == lengths[rid]:
                    book.release(rid)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gated_norm_kernel(dtype):
    from mrun_b200.kernels import ops
    act = torch.float32 if dtype == "float32" else torch.bfloat16
    gen = torch.Generator().manual_seed(8)
    for groups, n, shared in ((1, 120, False), (6, 20, True), (3, 33, True), (4, 128, False), (1, 2050, False), (2, 1024, True)):
        o = (torch.randn(9, groups * n, generator=gen) * 3).to(DEV)
        wide = torch.randn(9, groups * n + 16, generator=gen).to(DEV, act)
        gate = wide[:, 16:]
        weight = (1 + 0.3 * torch.randn(n if shared else groups * n, generator=gen)).to(DEV)
        got = ops.gated_norm(o, weight, gate, 1e-5, groups, act)
        x = o.cpu().double().view(9, groups, n)
        w = weight.cpu().double().view(1, 1, n) if shared else weight.cpu().double().view(1, groups, n)
        want = x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * w * torch.sigmoid(gate.cpu().double().view(9, groups, n))
        close(got, want.view(9, -1), dtype, f"{groups} groups of {n}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_table_route_and_clamped_glu_kernels(dtype):
    from mrun_b200.kernels import ops
    act = torch.float32 if dtype == "float32" else torch.bfloat16
    gen = torch.Generator().manual_seed(3)
    for experts, top, ff in ((2, 1, 8), (5, 3, 11), (8, 8, 16), (40, 2, 24)):
        table = torch.rand(50, experts, generator=gen).argsort(1)[:, :top].to(torch.int32)
        ids = torch.randint(0, 50, (21,), generator=gen).to(torch.int32)
        chosen = torch.empty(21, top, dtype=torch.int32, device=DEV)
        weights = ops.table_route(ids.to(DEV), table.to(DEV), experts, chosen=chosen)
        want = torch.zeros(21, experts)
        want.scatter_(1, table[ids.long()].long(), 1.0 / top)
        assert torch.equal(weights.cpu(), want) and torch.equal(chosen.cpu(), table[ids.long()])
        u = (torch.randn(21, experts * 2 * ff, generator=gen) * 2).to(DEV, act)
        got = ops.clamped_glu(u, weights, experts, ff, 1.25, 1.702)
        v = u.cpu().double().view(21, experts, 2, ff)
        g, up = v[:, :, 0].clamp(max=1.25), v[:, :, 1].clamp(-1.25, 1.25)
        full = g * torch.sigmoid(1.702 * g) * (up + 1)
        close(got, (full * want.double()[:, :, None]).view(21, -1), dtype, "weights per expert")
        row_weight = torch.rand(21, generator=gen).to(DEV)
        got = ops.clamped_glu(u[:, :2 * ff].contiguous(), row_weight, 1, ff, 1.25, 1.702)
        close(got, full[:, 0] * row_weight.cpu().double()[:, None], dtype, "a weight per row")


# ------------------------------------------------------------------ mixers alone

def random_tensors(specs, prefix, gen, std=0.3):
    out = {}
    for t in specs:
        name = t.name[len(prefix) + 1:]
        if t.init == "norm":
            out[name] = 1 + 0.2 * torch.randn(t.shape, generator=gen)
        elif t.init == "log_rate":
            out[name] = torch.rand(t.shape, generator=gen) * 3 - 3
        else:
            out[name] = torch.randn(t.shape, generator=gen) * std
        out[name] = out[name].to(torch.bfloat16).float()           # values both precisions hold exactly
    return out


LENGTHS = {"a": 75, "b": 2, "c": 140, "d": 1, "e": 37}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads, dim, vdim", [(3, 16, 40), (2, 72, 33), (1, 160, 16), (5, 32, 32), (2, 128, 64)])
def test_decay_attention_alone(dtype, heads, dim, vdim):
    from mrun_b200.config.spec import DecayAttentionSpec
    from mrun_b200.parts import MIXERS
    rt = runtime(dtype)
    decay = tuple(np.linspace(0.4, 0.999, heads).tolist())
    spec = DecayAttentionSpec(hidden=48, heads=heads, dim=dim, vdim=vdim, decay=decay, eps=1e-5)
    w = random_tensors(MIXERS.tensor_specs(spec, "m"), "m", torch.Generator().manual_seed(heads))
    part = MIXERS.build(spec, w, rt)
    named = {f"m.{k}": v.double() for k, v in w.items()}
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    check_mixer(part, 48, dtype, LENGTHS, lambda h: plain.lightning(h, named, "m", m, 1e-5), rt=rt)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, conv", [(4, 2, 16, 24, 4), (2, 1, 40, 70, 2), (3, 3, 128, 8, 3),
                                                              (6, 2, 24, 20, 5), (1, 1, 160, 32, 2)])
def test_channel_delta_alone(dtype, heads, kv_heads, dim, vdim, conv):
    from mrun_b200.config.spec import ChannelDeltaSpec
    from mrun_b200.parts import MIXERS
    rt = runtime(dtype)
    spec = ChannelDeltaSpec(hidden=56, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv, decay_rank=8,
                            gate_rank=5, eps=1e-5)
    w = random_tensors(MIXERS.tensor_specs(spec, "m"), "m", torch.Generator().manual_seed(dim))
    part = MIXERS.build(spec, w, rt)
    named = {f"m.{k}": v.double() for k, v in w.items()}
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}
    check_mixer(part, 56, dtype, LENGTHS, lambda h: plain.channel_delta(h, named, "m", m, 1e-5), rt=rt,
                bound=None if dtype == "float32" else 4e-2)


ATTENTION_SHAPES = [  # heads, kv heads, key size, value size, rotating features, page size
    (6, 3, 16, 32, 8, 16),       # bfloat16: two value chunks through the mma.sync kernels
    (5, 5, 20, 28, 20, 8),       # CUDA-core kernel
    (4, 1, 12, 36, 0, 4),
    (4, 2, 64, 64, 16, 16),      # bfloat16: TMA decode and tcgen05 prefill kernels, one chunk
    (2, 1, 64, 128, 64, 8),      # the same, two chunks
    (3, 1, 128, 128, 32, 16),    # the same kernels at 128
    (34, 2, 16, 16, 4, 16),      # seventeen query heads a kv head: beyond the decode kernels' groups
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, rot, page", ATTENTION_SHAPES)
def test_differential_attention_alone(dtype, heads, kv_heads, dim, vdim, rot, page):
    from mrun_b200.config.spec import DifferentialAttentionSpec, ScaledRotarySpec
    from mrun_b200.parts import MIXERS
    rt = runtime(dtype, page)
    position = ScaledRotarySpec(dims=rot, base=300.0, pairing="half") if rot else None
    spec = DifferentialAttentionSpec(hidden=40, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, softmax_scale=0.3,
                                     diff=0.3, eps=1e-5, position=position)
    w = random_tensors(MIXERS.tensor_specs(spec, "m"), "m", torch.Generator().manual_seed(dim + vdim))
    part = MIXERS.build(spec, w, rt)
    named = {f"m.{k}": v.double() for k, v in w.items()}
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": 0.3, "diff": 0.3,
         "rot": {"dims": rot, "base": 300.0}}

    def fn(h):
        return plain.differential_attention(h, named, "m", m, 1e-5, torch.arange(h.shape[0]))
    check_mixer(part, 40, dtype, LENGTHS, fn, rt=rt)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim, vdim, page", [(16, 32, 16), (20, 28, 8), (64, 64, 16)])
def test_differential_attention_one_key_stands_out(dtype, dim, vdim, page):
    """One far key and the queries that look for it are scaled so that its score dominates one map
    of one head: at the first token, on both sides of a page border and hundreds of tokens back,
    asked for from inside a prompt portion and by tokens decoded alone.  Losing that key, or
    taking the one beside it, changes the head's output by about its size."""
    from mrun_b200.config.spec import DifferentialAttentionSpec, ScaledRotarySpec
    from mrun_b200.parts import MIXERS
    rt = runtime(dtype, page)
    hidden, heads = 32, 2
    spec = DifferentialAttentionSpec(hidden=hidden, heads=heads, kv_heads=1, dim=dim, vdim=vdim, softmax_scale=0.5,
                                     diff=0.2, eps=1e-5, position=ScaledRotarySpec(dims=8, base=50.0, pairing="half"))
    gen = torch.Generator().manual_seed(17)
    w = random_tensors(MIXERS.tensor_specs(spec, "m"), "m", gen, std=0.1)
    # the last (unrotated) feature of map 1 of both heads, and of the key's map 1, reads input column 0 alone
    # (the key reads column 0, the queries column 1, so that an asking token is no such key itself)
    w["q"][:, :2] = 0; w["k"][:, :2] = 0
    for row in (dim - 1, 2 * dim + dim - 1):
        w["q"][row] = 0; w["q"][row, 1] = 1
    w["k"][dim - 1] = 0; w["k"][dim - 1, 0] = 1
    part = MIXERS.build(spec, w, rt)
    named = {f"m.{k}": v.double() for k, v in w.items()}
    m = {"heads": heads, "kv_heads": 1, "dim": dim, "vdim": vdim, "scale": 0.5, "diff": 0.2, "rot": {"dims": 8, "base": 50.0}}
    total = 420
    for far in (0, page - 1, page, 2 * page + 1, 100):
        x = torch.randn(total, hidden, generator=gen) * 0.5
        x[:, 0] = 0
        x[far, 0] = 8.0                                     # the key
        askers = [far + 1, far + page, 300, 401, 419]       # in the prompt portion and decoded alone
        x[askers, 1] = 8.0                                  # score 64 * 0.5 above all others
        want = plain.differential_attention(x.to(rt.precision.act).double(), named, "m", m, 1e-5, torch.arange(total))
        lost = x.clone(); lost[far, 0] = 0
        blind = plain.differential_attention(lost.to(rt.precision.act).double(), named, "m", m, 1e-5, torch.arange(total))
        assert float((want - blind)[askers].abs().max(1).values.min() / want.abs().max()) > 0.2     # every asker sees the key
        book = Steps(part.cache_need(), rt, pages=-(-total // page) + 2, slots=1)
        got = []
        for n in [400] + [1] * 20:
            def run(ctx, places):
                (_, start, _, count), = places
                return part.forward(x[start:start + count].to(DEV, rt.precision.act), ctx, book.cache).float().cpu()
            got.append(book.run([("r", n)], run))
        got = torch.cat(got)
        close(got[askers], want[askers], dtype, f"key at {far}")
        close(got, want, dtype, f"key at {far}, all tokens")
        book.release("r")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("experts, top, ff", [(5, 3, 40), (3, 1, 22), (4, 4, 16), (16, 2, 24)])
def test_table_routed_alone(dtype, experts, top, ff, monkeypatch):
    """Rows alone against rows in a batch, and the sorted path against the path that computes every expert."""
    from mrun_b200.config.spec import TableRoutedMLPSpec
    from mrun_b200.parts import FEED_FORWARDS, routed
    rt = runtime(dtype)
    hidden, vocab = 64, 90
    spec = TableRoutedMLPSpec(hidden=hidden, vocab=vocab, experts=experts, top=top, expert_ff=ff, limit=1.5)
    gen = torch.Generator().manual_seed(experts)
    w = random_tensors([t for t in FEED_FORWARDS.tensor_specs(spec, "f") if not t.name.endswith("table")], "f", gen, std=0.3)
    w["table"] = torch.rand(vocab, experts, generator=gen).argsort(1)[:, :top].to(torch.int32)
    part = FEED_FORWARDS.build(spec, w, rt)
    named = {f"f.{k}": (v.double() if v.is_floating_point() else v) for k, v in w.items()}
    ids = torch.randint(0, vocab, (45,), generator=gen)
    x = torch.randn(45, hidden, generator=gen).to(rt.precision.act)
    mlp = {"router": {"experts": experts, "top": top}, "expert": {"limit": 1.5}}
    want = plain.table_moe(x.double(), named, "f", mlp, ids.tolist())

    class Ctx:
        token_ids = ids.to(DEV, torch.int32)
    monkeypatch.setattr(routed, "SORT_MIN_SAVED_FLOPS", 1e30)
    got = part.forward(x.to(DEV), Ctx)
    close(got, want, dtype, "every expert computed")
    Ctx.token_ids = ids[7:8].to(DEV, torch.int32)
    alone = part.forward(x[7:8].to(DEV), Ctx)
    if dtype == "float32":
        assert torch.equal(alone[0], got[7])
    close(alone, want[7:8], dtype, "a row alone")
    if dtype == "bfloat16" and top < experts:
        monkeypatch.setattr(routed, "SORT_MIN_SAVED_FLOPS", 0.0)
        Ctx.token_ids = ids.to(DEV, torch.int32)
        close(part.forward(x.to(DEV), Ctx), want, dtype, "sorted by expert")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("streams, taps, with_ff", [(3, 4, True), (0, 0, True), (1, 2, False), (4, 5, True)])
def test_streams_block_alone(dtype, streams, taps, with_ff):
    """A layer under several streams with an input convolution: the streams after the layer's
    last write, fed whole and in portions."""
    from mrun_b200.config.spec import DecayAttentionSpec, GatedMLPSpec, LayerSpec, RMSNormSpec
    from mrun_b200.kernels import ops
    from mrun_b200.parts import ARRANGEMENTS
    rt = runtime(dtype)
    width, count = 48, max(1, streams)
    norm = RMSNormSpec(width, 1e-5, bare=True, scalar=True)
    mixer = DecayAttentionSpec(hidden=width, heads=2, dim=16, vdim=24, decay=(0.7, 0.95), eps=1e-5)
    spec = LayerSpec(prefix="b", mixer=mixer, feed_forward=GatedMLPSpec(width, 64, "silu", ("gate", "up", "down")) if with_ff else None,
                     mixer_norm=norm, feed_forward_norm=norm if with_ff else None, arrangement="streams", mixer_prefix="mix",
                     feed_forward_prefix="mlp", mixer_norm_prefix="norm1", feed_forward_norm_prefix="norm2",
                     streams=streams, input_conv_taps=taps)
    cls = ARRANGEMENTS.get("streams")
    gen = torch.Generator().manual_seed(streams + taps)
    w = {}
    for t in cls.tensor_specs(spec):
        if t.init == "streams_in":
            w[t.name] = 1.0 / count + 0.2 * torch.randn(t.shape, generator=gen)
        elif t.init == "streams_mix":
            w[t.name] = torch.eye(count) + 0.2 * torch.randn(t.shape, generator=gen)
        elif t.init == "norm":
            w[t.name] = 1 + 0.2 * torch.randn(t.shape, generator=gen)
        else:
            w[t.name] = torch.randn(t.shape, generator=gen) * 0.3
        w[t.name] = w[t.name].to(torch.bfloat16).float()
    block = cls(spec, w, rt)
    wd = {k: v.double() for k, v in w.items()}
    total = 50
    x0 = torch.randn(total, count, width, generator=gen)
    m = {"heads": 2, "dim": 16, "vdim": 24, "decay": [0.7, 0.95]}

    def mix(h):
        if taps:
            h = h + plain.causal_conv(h, wd["b.canon1"])
        return plain.lightning(h, wd, "b.mix", m, 1e-5)
    s = x0.double().permute(1, 0, 2)
    if streams:
        s = plain.hyper_step(s, wd, "b.hc1", mix, wd["b.norm1"], 1e-5)
        if with_ff:
            s = plain.hyper_step(s, wd, "b.hc2", lambda h: plain.dense_ff(h, wd, "b.mlp"), wd["b.norm2"], 1e-5)
    else:
        s = s + mix(plain.rms_norm(s[0], wd["b.norm1"], 1e-5))[None]
        if with_ff:
            s = s + plain.dense_ff(plain.rms_norm(s[0], wd["b.norm2"], 1e-5), wd, "b.mlp")[None]
    want = s.permute(1, 0, 2)
    for chunks in ([total], [2, 1, 30, 17]):
        book = Steps(block.cache_need(), rt, slots=1)
        got = []
        for n in chunks:
            def run(ctx, places):
                (_, start, _, count_), = places
                resid = x0[start:start + count_].reshape(count_, -1).to(DEV)
                pending = block.forward(resid, None, ctx, book.cache)
                assert isinstance(pending, ops.PendingStreams)
                ops.streams_step(resid, pending, None, None, 0.0, torch.float32, count, want_sum=True)
                return resid.cpu()
            got.append(book.run([("r", n)], run))
        close(torch.cat(got).view(total, count, width), want, dtype, f"streams after the layer, fed as {chunks}",
              bound=None if dtype == "float32" else 2e-2)


# ------------------------------------------------------------------ whole models, cut in every way

TRACE_LENGTHS = [70, 1, 133, 2, 45, 260, 97, 3, 161]
SIZES = [2, 7, 3, 16, 5, 2, 33, 9, 64, 4, 1]


@pytest.fixture(scope="module", params=sorted(BTINY))
def btiny(request, tmp_path_factory):
    name = request.param
    return name, make_folder(name, str(tmp_path_factory.mktemp(f"balivik_{name}"))), BTINY[name]


# bfloat16 bound of whole models, relative to the largest plain logit.  Measured: V, W and X stay
# under 4e-2; U (eight layer runs over two streams, unit-length keys feeding a delta rule) reaches
# 9e-2 in both attention paths alike, layer by layer from 1e-2 after its first layer: rounding, not
# a path (every mechanism alone is held to 3e-2 above, every cutting in 32-bit to equal bits).
BF16_MODEL_BOUND = 0.12


@pytest.mark.parametrize("dtype, sorted_experts, tensor_core_maps",
                         [("float32", False, True), ("bfloat16", False, True), ("bfloat16", True, True),
                          ("bfloat16", False, False)])
def test_every_cutting_matches_plain(btiny, dtype, sorted_experts, tensor_core_maps, tmp_path, monkeypatch):
    """``sorted_experts``: steps of more than 16 rows sort their rows by expert and compute the
    chosen experts only; ``tensor_core_maps``: the differential attention's maps go through the
    tensor-core attention kernels where they take the shape, else one CUDA-core kernel runs both."""
    name, folder, settings = btiny
    cfg, weights = load_folder(folder)
    vocab = cfg["vocab"]
    requests = {f"r{i}": tokens_of(vocab, n, seed=200 + i) for i, n in enumerate(TRACE_LENGTHS)}
    want = {rid: plain.forward(cfg, weights, tokens).to(torch.float32).numpy() for rid, tokens in requests.items()}
    cuts = {}
    b = TraceBuilder()

    def section(label):
        cuts[label] = len(b.where)
    section("whole")
    for rid in ("r0", "r1", "r3", "r5"):
        cut_whole(b, rid, requests[rid])
    section("decode_tail")
    cut_decode_tail(b, "r0", requests["r0"])
    cut_decode_tail(b, "r7", requests["r7"], tail=2)
    cut_decode_tail(b, "r5", requests["r5"], tail=200 if name == "U" else 40)          # long decoding
    section("portions")
    for k, rid in enumerate(("r2", "r4", "r5", "r3")):
        cut_portions(b, rid, requests[rid], SIZES[k:] + SIZES[:k])
    section("mixed")
    cut_mixed(b, requests, SIZES, live=4, seed=6)
    section("end")
    # four live requests, each rounded up to 64 tokens: so few pages and slots that they are used again
    rounded = sorted((-(-n // 64) * 64 for n in TRACE_LENGTHS), reverse=True)
    monkeypatch.setenv("MRUN_MOE_SORT_MIN_FLOPS", "0" if sorted_experts else "1e30")
    monkeypatch.setenv("MRUN_DIFF_TENSOR_CORE", "1" if tensor_core_maps else "0")
    runner = TraceRunner(folder, dtype, str(tmp_path / "out"), sum(rounded[:4]), settings["page_size"], max_requests=4)
    try:
        runner.run(b.steps)
    finally:
        assert runner.close() == 0
    scale = max(float(np.max(np.abs(w))) for w in want.values())
    bound = 2e-5 if dtype == "float32" else BF16_MODEL_BOUND
    files, worst, first_seen = {}, {}, {}
    labels = list(cuts)
    for index, (step, row, rid, position) in enumerate(b.where):
        if step not in files:
            files[step] = runner.logits(step, vocab)
        got = files[step][row]
        if dtype == "float32":
            seen = first_seen.setdefault((rid, position), (got, step))
            assert np.array_equal(seen[0], got), (f"{name}: request {rid}, position {position}: steps {seen[1]} and "
                                                  f"{step} differ in bits")
        error = float(np.max(np.abs(got - want[rid][position]))) / scale
        label = [l for l in labels[:-1] if cuts[l] <= index][-1]
        if error > worst.get(label, (0.0,))[0]:
            worst[label] = (error, step, rid, position)
    print(name, dtype, sorted_experts, tensor_core_maps, {k: f"{v[0]:.2e}" for k, v in worst.items()})
    for label, (error, step, rid, position) in worst.items():
        assert error <= bound, f"{name}/{dtype}/{label}: error {error:.3e} at step {step}, request {rid}, position {position}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_matches_plain(btiny, dtype):
    from mrun_b200 import Engine
    name, folder, settings = btiny
    cfg, weights = load_folder(folder)
    prompts = [tokens_of(cfg["vocab"], n, seed=300 + n) for n in (1, 9, 40, 71, 5)]
    engine = Engine.from_folder(folder, dtype=dtype, page_size=settings["page_size"], context=512,
                                max_batch_tokens=7, max_requests=4)
    results = engine.generate(prompts, max_tokens=10, ignore_eos=True)
    assert engine.executor.model.graph_safe and engine.executor._graphs          # decoding ran as captured steps
    for prompt, result in zip(prompts, results):
        assert result.finish_reason == "length" and len(result.tokens) == 10
        tokens = list(prompt)
        for n, token in enumerate(result.tokens):
            logits = plain.forward(cfg, weights, tokens)[-1]
            best = int(torch.argmax(logits))
            margin = 1e-3 if dtype == "float32" else 2 * BF16_MODEL_BOUND * float(logits.abs().max())
            assert token == best or float(logits[best] - logits[token]) < margin, \
                f"{name}: output token {n}: engine {token}, plain {best}, behind by {float(logits[best] - logits[token]):.4f}"
            tokens.append(token)
    engine.executor.cache.check_invariants()
    assert not engine.executor.cache.live


def test_preempted_requests_start_from_a_cleared_state(tmp_path):
    """Pages taken on demand from a pool that runs out: the request admitted last gives its pages
    and its state slot back and is fed again from its first token; its recurrent and convolution
    states must then start from zero, or its later tokens differ from a run with room enough."""
    from mrun_b200 import Engine
    folder = make_folder("U", str(tmp_path / "u"))          # attention layers (pages) beside both recurrent kinds
    cfg, weights = load_folder(folder)
    prompts = [tokens_of(cfg["vocab"], n, seed=400 + n) for n in (20, 25, 30, 18)]
    roomy = Engine.from_folder(folder, dtype="float32", page_size=16, context=1024, max_batch_tokens=32, max_requests=4)
    want = [r.tokens for r in roomy.generate(prompts, max_tokens=40, ignore_eos=True)]
    pool = Engine.from_folder(folder, dtype="float32", page_size=16, num_pages=10, max_batch_tokens=32, max_requests=4,
                              reserve=False)
    got = pool.generate(prompts, max_tokens=40, ignore_eos=True)
    assert pool.stats.preemptions > 0, "the pool was meant to run out"
    for prompt, run, tokens in zip(prompts, got, want):
        if run.tokens != tokens:                    # a near-tie may fall the other way: ask the plain model
            fed = list(prompt)
            for token in run.tokens:
                logits = plain.forward(cfg, weights, fed)[-1]
                best = int(torch.argmax(logits))
                assert token == best or float(logits[best] - logits[token]) < 1e-3
                fed.append(token)
    pool.executor.cache.check_invariants()
    assert pool.executor.cache.free_pages() == pool.executor.cache.num_pages


def test_command_line_random_then_run(tmp_path):
    """``mrun random`` writes a Balivik folder from its config.json, ``mrun run`` generates from it."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), os.pardir))
    mrun = os.path.join(root, "bin", "mrun")
    run = lambda *args: subprocess.run([sys.executable, mrun, *args], capture_output=True, text=True, timeout=600)
    (tmp_path / "cfg.json").write_text(json.dumps(BTINY["X"]["config"]))
    folder = str(tmp_path / "model")
    made = run("random", folder, "--config", str(tmp_path / "cfg.json"), "--seed", "21", "--std", "0.1")
    assert made.returncode == 0, made.stderr
    cfg, weights = load_folder(folder)
    prompt = tokens_of(cfg["vocab"], 19, seed=8)
    result = run("run", folder, "--prompt", ",".join(map(str, prompt)), "--max-tokens", "6", "--dtype", "float32",
                 "--ignore-eos", "--context", "1K")
    assert result.returncode == 0, result.stderr
    tokens = list(prompt)
    for token in (int(t) for t in result.stdout.strip().split(",")):
        logits = plain.forward(cfg, weights, tokens)[-1]
        best = int(torch.argmax(logits))
        assert token == best or float(logits[best] - logits[token]) < 1e-3
        tokens.append(token)
    assert len(tokens) == 19 + 6 and "Balivik" in result.stderr


# ------------------------------------------------------------------ layer sizes of a real model

REAL_SIZES = {"architecture": "Balivik", "vocab": 4096, "width": 1024, "norm": {"eps": 1e-6}, "streams": 4,
              "canon": {"taps": 4}, "logit_scale": 0.5,
              "layers": [
                  {"type": "channel_delta", "mlp": {"kind": "dense", "ff": 2048},
                   "mixer": {"heads": 8, "kv_heads": 8, "dim": 128, "vdim": 128, "conv": 4, "decay_rank": 64, "gate_rank": 64}},
                  {"type": "attention", "mlp": {"kind": "moe", "router": {"experts": 8, "top": 2}, "expert": {"ff": 512, "limit": 7.0}},
                   "mixer": {"heads": 8, "kv_heads": 2, "dim": 128, "vdim": 256, "scale": 128 ** -0.5, "diff": 0.3,
                             "rot": {"base": 10000.0, "dims": 64}}},
                  {"type": "lightning", "mlp": {"kind": "dense", "ff": 2048},
                   "mixer": {"heads": 8, "dim": 128, "vdim": 128, "decay": [1 - 2.0 ** -(2 + i) for i in range(8)]}}]}


@pytest.mark.parametrize("dtype, sorted_experts", [("float32", False), ("bfloat16", False), ("bfloat16", True)])
def test_real_layer_sizes(dtype, sorted_experts, tmp_path, monkeypatch):
    """Heads of 128 x 128 (full row slices of the scans), attention keys of 128 with values of 256
    (two chunks through the tcgen05 and TMA kernels), four streams of 1,024, experts of 512: a
    prompt whole and in portions, then decoded token by token, against the plain model."""
    from mrun_b200.config.balivik import BalivikConfig
    from mrun_b200.engine import StepEntry
    from mrun_b200.engine.loading import executor_from_folder
    from mrun_b200.parts import routed
    from mrun_b200.weights import write_random_model
    monkeypatch.setattr(routed, "SORT_MIN_SAVED_FLOPS", 0.0 if sorted_experts else 1e30)
    folder = write_random_model(BalivikConfig.from_dict(REAL_SIZES), str(tmp_path / "real"), seed=7, std=0.03, norm_noise=0.1)
    cfg, weights = load_folder(folder)
    tokens = tokens_of(cfg["vocab"], 330, seed=77)
    want = plain.forward(cfg, weights, tokens).to(torch.float32)
    ex = executor_from_folder(folder, dtype=dtype, page_size=16, num_pages=64, max_requests=2)
    seen = {}
    for label, portions in (("whole", [330]), ("portions", [200, 3, 65, 30] + [1] * 32)):
        request, at, got = ex.admit(label), 0, []
        for n in portions:
            got.append(ex.step([StepEntry(request, tokens[at:at + n], list(range(n)))]).cpu())
            at += n
        ex.release(request)
        got = torch.cat(got)
        error = float((got - want).abs().max() / want.abs().max())
        print(dtype, sorted_experts, label, f"{error:.2e}")
        assert error <= (2e-5 if dtype == "float32" else BF16_MODEL_BOUND), f"{label}: {error:.3e}"
        if dtype == "float32":
            assert torch.equal(seen.setdefault("logits", got), got), "the cuttings differ in bits"
    ex.check()
