"""Zasesun on the GPU against the plain implementation (``plain_zasesun``): every mechanism alone,
then whole models replayed through ``bin/trace_run`` cut in every way, then greedy generation
through ``Engine.generate``."""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import plain_zasesun as plain
from tiny_zasesun import ZTINY, load_folder, make_folder, tokens_of
from trace_tools import TraceBuilder, TraceRunner, cut_decode_tail, cut_mixed, cut_portions, cut_whole

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


def runtime(dtype, page_size=8):
    from mrun_b200.parts import Precision, Runtime
    return Runtime(torch.device(DEV), Precision.of(dtype), page_size)


def tolerance(dtype):
    return 3e-5 if dtype == "float32" else 3e-2


def steps_of_one_request(needs, total, rt, chunks, pages=64):
    """A cache manager for the given needs and the step contexts of one request of ``total``
    tokens fed in the given chunk sizes."""
    from mrun_b200.cache import CacheManager
    from mrun_b200.engine.batch import HostStaging, StepEntry, build_context
    manager = CacheManager(needs, [None] * len(needs), rt.page_size, pages, 2, device=rt.device, dtype=rt.precision.act)
    staging = HostStaging(rt.device)
    request = manager.admit("r")
    for n in chunks:
        start = request.length
        plan = manager.plan_append([(request, n)])
        ctx = build_context([StepEntry(request, [0] * n)], manager, staging)
        yield ctx, manager, start, n
        manager.commit(plan)
    assert request.length == total


def close(got, want, dtype, what="", bound=None):
    got, want = got.detach().to("cpu", F64), want.to(F64)
    error = float((got - want).abs().max() / want.abs().max())
    assert error <= (bound or tolerance(dtype)), f"{what}: relative error {error:.3e}"


# ------------------------------------------------------------------ kernels alone

@pytest.mark.parametrize("scaling", [None, (4.0, 64.0, 4.0, 1.0), (1.5, 300.0, 16.0, 0.25)])
def test_scaled_rotary_table(scaling):
    from mrun_b200.config import ScaledRotarySpec
    from mrun_b200.parts import POSITIONS
    rt = runtime("float32")
    part = POSITIONS.build(ScaledRotarySpec(dims=12, base=16.0, pairing="interleaved", scaling=scaling), {}, rt)
    rot = {"dims": 12, "base": 16.0}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    freq, magnitude = plain.rotary_frequencies(rot)
    for ctx, _, start, n in steps_of_one_request([], 700, rt, [690, 10], pages=100):
        table = part.rotation(ctx).cpu().double()
        assert part.rotation(ctx) is not None and table.shape == (n, 6, 2)
        angle = torch.arange(start, start + n, dtype=F64)[:, None] * freq[None, :]
        assert (table[..., 0] - torch.cos(angle) * magnitude).abs().max() < 2e-7
        assert (table[..., 1] - torch.sin(angle) * magnitude).abs().max() < 2e-7


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_post_norm_add_kernel(dtype):
    from mrun_b200.kernels import ops
    act = torch.float32 if dtype == "float32" else torch.bfloat16
    for hidden in (100, 256, 1000):
        stream = torch.randn(9, hidden, device=DEV)
        branch = torch.randn(9, hidden, device=DEV) * 3
        w_post, w_next = (1 + 0.2 * torch.randn(hidden, device=DEV) for _ in range(2))
        want_stream = stream.cpu().double() + 0.6 * plain.rms_norm(branch.cpu().double(), w_post.cpu().double(), 1e-3)
        want = plain.rms_norm(want_stream, w_next.cpu().double(), 1e-5)
        rows = torch.tensor([8, 0, 3], dtype=torch.int32, device=DEV)
        picked = torch.empty(3, hidden, dtype=act, device=DEV)
        before = stream.clone()
        ops.post_norm_add(stream, branch, w_post, 0.6, 1e-3, w_next, 1e-5, picked, rows=rows)
        assert torch.equal(stream, before)                       # with rows the stream stays
        close(picked, want[[8, 0, 3]], dtype, "rows")
        out = torch.empty(9, hidden, dtype=act, device=DEV)
        ops.post_norm_add(stream, branch, w_post, 0.6, 1e-3, w_next, 1e-5, out)
        close(out, want, dtype, "normed")
        close(stream, want_stream, "float32", "stream")          # the stream is 32-bit in both precisions
        same = stream.clone()
        ops.post_norm_add(same, torch.zeros_like(branch), w_post, 0.6, 1e-3, None, 0.0, None)
        assert torch.equal(same, stream)


def test_route_top_k_kernel():
    from mrun_b200.kernels import ops
    gen = torch.Generator().manual_seed(4)
    for experts, top in ((3, 1), (8, 4), (5, 5), (70, 6), (512, 8)):
        logits = (torch.randn(33, experts, generator=gen) * 2).to(DEV)
        chosen = torch.empty(33, top, dtype=torch.int32, device=DEV)
        got = ops.route_top_k(logits, top, "softmax", False, chosen=chosen).cpu().double()
        scores = torch.softmax(logits.cpu().double(), -1)
        order = torch.topk(scores, top, dim=-1).indices
        want = torch.zeros_like(scores).scatter(1, order, scores.gather(1, order))
        assert (got - want).abs().max() < 1e-6
        assert torch.equal(chosen.cpu().long(), order)           # picked in falling order of score
        got = ops.route_top_k(logits, top, "sigmoid", True).cpu().double()
        scores = torch.sigmoid(logits.cpu().double())
        order = torch.topk(scores, top, dim=-1).indices
        kept = scores.gather(1, order)
        want = torch.zeros_like(scores).scatter(1, order, kept / kept.sum(-1, keepdim=True))
        assert (got - want).abs().max() < 1e-6
    # equal scores: the smaller index wins
    got = ops.route_top_k(torch.zeros(2, 6, device=DEV), 2).cpu()
    assert torch.equal(got != 0, torch.tensor([[True, True, False, False, False, False]] * 2))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_relu2_soft_cap_and_per_head_products(dtype):
    from mrun_b200.kernels import ops
    act = torch.float32 if dtype == "float32" else torch.bfloat16
    u = torch.randn(11, 3 * 7 + 5, device=DEV).to(act)
    weights = torch.rand(11, 3, device=DEV)
    got = ops.relu2_scaled(u, weights, 3, 7)
    factor = torch.cat([weights.cpu().double().repeat_interleave(7, dim=1), torch.ones(11, 5, dtype=F64)], dim=1)
    close(got, torch.relu(u.cpu().double()) ** 2 * factor, dtype, "relu2 with weights")
    close(ops.relu2_scaled(u, None, 0, 1), torch.relu(u.cpu().double()) ** 2, dtype, "relu2 alone")
    wide = torch.randn(300, 5 * 16 + 24, device=DEV).to(act)          # eight columns a thread
    wide_weights = torch.rand(300, 5, device=DEV)
    factor = torch.cat([wide_weights.cpu().double().repeat_interleave(16, dim=1), torch.ones(300, 24, dtype=F64)], dim=1)
    close(ops.relu2_scaled(wide, wide_weights, 5, 16), torch.relu(wide.cpu().double()) ** 2 * factor, dtype, "relu2, wide rows")
    x = torch.randn(6, 50, device=DEV) * 20
    close(ops.soft_cap(x.clone(), 7.0), plain.soft_cap(x.cpu().double(), 7.0), "float32", "soft cap")
    # heads side by side in wider rows, in and out
    for tokens in (1, 5, 130):
        heads, k, n = 3, 20, 9
        rows_in = torch.randn(tokens, heads, k + 4, device=DEV).to(act)
        w = torch.randn(heads, n, k, device=DEV).to(act)
        rows_out = torch.full((tokens, heads, n + 3), 7.0, device=DEV).to(act)
        ops.linear_per_head(rows_in[:, :, :k], w, rows_out[:, :, :n])
        want = torch.einsum("thk,hnk->thn", rows_in[:, :, :k].cpu().double(), w.cpu().double())
        close(rows_out[:, :, :n], want, dtype, f"per-head product of {tokens} rows")
        assert bool((rows_out[:, :, n:] == 7.0).all())


def test_which_rows_the_wide_kernel_takes():
    from mrun_b200.kernels.attention import latent_wide_ok, supports_tensor_cores
    assert latent_wide_ok(torch.bfloat16, 576, 512) and latent_wide_ok(torch.bfloat16, 272, 264)
    assert not latent_wide_ok(torch.float32, 576, 512)          # the 32-bit path stays on CUDA cores
    assert not latent_wide_ok(torch.bfloat16, 1024, 600)        # more value columns than four warps hold
    assert not latent_wide_ok(torch.bfloat16, 568, 512)         # rows are padded to multiples of 16
    assert not supports_tensor_cores(torch.bfloat16, 272, 20)   # such rows are beyond the per-head-size kernels


# ------------------------------------------------------------------ parts alone

def random_part_tensors(specs, seed, std=0.15):
    from mrun_b200.weights.random_init import random_tensor
    return {t.name: random_tensor(t, seed, std, 0.2, torch.bfloat16) for t in specs}


MIXERS = {
    # heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rotary (dims, base, scaling)
    "row48": (2, 16, 8, 24, 24, 40, 0.4, (8, 100.0, None)),
    "row64": (3, 32, 16, 16, 40, 48, 0.3, (16, 500.0, (4.0, 64.0, 8.0, 2.0))),
    "row128": (4, 24, 16, 40, 56, 112, 0.3, (16, 10000.0, (2.0, 32.0, 4.0, 0.5))),
    "row272_20heads": (20, 8, 8, 8, 32, 264, 0.4, (8, 50.0, None)),
    "row576": (16, 24, 64, 16, 32, 512, 0.2, (64, 10000.0, (4.0, 256.0, 32.0, 1.0))),
    "row304_3heads": (3, 16, 16, 24, 24, 280, 0.3, (16, 200.0, None)),
    "partly_rotated": (2, 16, 16, 8, 16, 24, 0.4, (8, 30.0, None)),
}


def build_mixer(name, dtype, page_size=8, seed=7):
    from mrun_b200.config import LatentAttentionSpec, ScaledRotarySpec
    from mrun_b200.parts import MIXERS as REGISTRY
    heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, (dims, base, scaling) = MIXERS[name]
    spec = LatentAttentionSpec(hidden=72, heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, q_rank=q_rank,
                               kv_rank=kv_rank, softmax_scale=scale, eps=1e-5,
                               position=ScaledRotarySpec(dims, base, "interleaved", scaling))
    rt = runtime(dtype, page_size)
    tensors = random_part_tensors(REGISTRY.tensor_specs(spec, "m"), seed)
    part = REGISTRY.build(spec, {k[2:]: v for k, v in tensors.items()}, rt)
    rot = {"dims": dims, "base": base}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    settings = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale, "rot": rot}
    return part, rt, tensors, settings


def run_mixer(part, rt, h, chunks):
    act = rt.precision.act
    outs = []
    for ctx, manager, start, n in steps_of_one_request([part.cache_need()], h.shape[0], rt, chunks, pages=128):
        outs.append(part.forward(h[start:start + n].to(DEV, act), ctx, manager.entries[0]).float().cpu())
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(MIXERS))
def test_latent_attention_part(name, dtype):
    """Whole, in portions down to one and two tokens, and token by token after a prompt."""
    part, rt, tensors, settings = build_mixer(name, dtype)
    gen = torch.Generator().manual_seed(1)
    h = torch.randn(75, 72, generator=gen).to(torch.bfloat16)
    want = plain.latent_attention(h.to(F64), tensors, "m", settings, 1e-5, torch.arange(75))
    whole = run_mixer(part, rt, h, [75])
    close(whole, want, dtype, "whole")
    for chunks in ([40, 2, 1, 17, 2, 13], [3] + [1] * 72, [1, 1, 2, 71]):
        cut = run_mixer(part, rt, h, chunks)
        close(cut, want, dtype, f"portions {chunks[:4]}")
        if dtype == "float32":
            assert torch.equal(cut, whole), "32-bit results must not depend on the cutting"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name, page_size", [("row64", 16), ("row128", 8), ("row48", 4), ("row272_20heads", 16),
                                             ("row576", 16), ("row304_3heads", 4)])
def test_one_key_stands_out(name, page_size, dtype):
    """The shared rotated key part is not normed, so a token whose input is scaled up has a key that
    dominates (or is shut out of) every head's softmax, wherever it sits: among the first tokens,
    on either side of a page's border, hundreds of tokens back.  A key that a kernel lost, or read
    from a neighbouring page, changes the result far beyond the tolerance."""
    part, rt, tensors, settings = build_mixer(name, dtype, page_size)
    length = 40 * page_size + 5
    gen = torch.Generator().manual_seed(2)
    for loud in (0, 1, page_size - 1, page_size, 3 * page_size - 1, 17 * page_size):
        h = torch.randn(length, 72, generator=gen)
        h[loud] *= 20.0
        h = h.to(torch.bfloat16)
        want = plain.latent_attention(h.to(F64), tensors, "m", settings, 1e-5, torch.arange(length))
        without = plain.latent_attention(torch.cat([h[:loud], h[loud + 1:]]).to(F64), tensors, "m", settings, 1e-5,
                                         torch.cat([torch.arange(loud), torch.arange(loud + 1, length)]))
        gap = float((want[-6:] - without[-6:]).abs().max() / want.abs().max())
        assert gap > 10 * tolerance(dtype), f"the loud key at {loud} does not show ({gap:.2e}): the test is too weak"
        # prompt, then the last tokens one by one, so that the key is far behind decoded tokens too
        got = run_mixer(part, rt, h, [length - 6, 2] + [1] * 4)
        # bfloat16: scores of a few hundred are rounded in steps of one or two, which moves the
        # weights of a softmax that the loud key does not quite own; a lost key moves the result
        # by more than half of its size (the gap above)
        close(got, want, dtype, f"loud key at {loud}", bound=None if dtype == "float32" else 0.1)
        assert gap > 0.3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("experts, top, shared", [(5, 2, 16), (3, 1, 0), (4, 4, 8), (40, 6, 0)])
def test_routed_feed_forward_part(experts, top, shared, dtype, monkeypatch):
    from mrun_b200.config import RoutedMLPSpec
    from mrun_b200.parts import FEED_FORWARDS, routed
    rt = runtime(dtype)
    spec = RoutedMLPSpec(hidden=72, experts=experts, top=top, expert_ff=24, shared_ff=shared)
    tensors = random_part_tensors(FEED_FORWARDS.tensor_specs(spec, "f"), 11, std=0.2)
    part = FEED_FORWARDS.build(spec, {k[2:]: v for k, v in tensors.items()}, rt)
    # in bfloat16 the step sorts its rows by expert and runs grouped products over the chosen ones
    monkeypatch.setattr(routed, "SORT_MIN_SAVED_FLOPS", 0.0)
    h = torch.randn(300, 72, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    mlp = {"router": {"experts": experts, "top": top}, "shared": {"ff": shared} if shared else None}
    want = plain.routed_feed_forward(h.to(F64), tensors, "f", mlp)
    got = part.forward(h.to(DEV, rt.precision.act), None)
    close(got, want, dtype, "all rows")
    assert part.sortable == (dtype == "bfloat16" and top < experts)
    again = part.forward(h.to(DEV, rt.precision.act), None)
    assert torch.equal(again, got), "the same step twice must give the same bits"
    if part.sortable:                  # and the step that computes every expert agrees
        monkeypatch.setattr(routed, "SORT_MIN_SAVED_FLOPS", 1e30)
        close(part.forward(h.to(DEV, rt.precision.act), None), want, dtype, "all rows, every expert computed")
        monkeypatch.setattr(routed, "SORT_MIN_SAVED_FLOPS", 0.0)
    for rows in ([0], [7, 8], list(range(20, 37))):               # a row's result is its own
        alone = part.forward(h[rows].to(DEV, rt.precision.act), None)
        close(alone, want[rows], dtype, f"rows {rows[:3]}")
        if dtype == "float32":
            assert torch.equal(alone, got[rows])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("with_feed_forward", [True, False])
def test_sandwich_block(with_feed_forward, dtype):
    from mrun_b200.config import GatedMLPSpec, LatentAttentionSpec, LayerSpec, RMSNormSpec, ScaledRotarySpec
    from mrun_b200.kernels import ops
    from mrun_b200.parts import ARRANGEMENTS
    rt = runtime(dtype)
    norm = RMSNormSpec(72, 1e-4, bare=True)
    mix = LatentAttentionSpec(hidden=72, heads=2, dim=16, rot_dim=8, vdim=24, q_rank=24, kv_rank=40, softmax_scale=0.4,
                              eps=1e-4, position=ScaledRotarySpec(8, 100.0, "interleaved", None))
    ff = GatedMLPSpec(72, 88, "gelu_tanh", tensor_names=("gate", "up", "down")) if with_feed_forward else None
    spec = LayerSpec(prefix="b", mixer=mix, feed_forward=ff, mixer_norm=norm, feed_forward_norm=norm if ff else None,
                     arrangement="sandwich", mixer_prefix="mix", feed_forward_prefix="mlp", mixer_norm_prefix="norm1",
                     feed_forward_norm_prefix="norm2", mixer_post_norm=norm, feed_forward_post_norm=norm if ff else None,
                     mixer_post_norm_prefix="norm1b", feed_forward_post_norm_prefix="norm2b", residual_scale=0.3)
    block_cls = ARRANGEMENTS.get("sandwich")
    tensors = random_part_tensors(block_cls.tensor_specs(spec), 13)
    block = block_cls(spec, tensors, rt)
    x = torch.randn(30, 72, generator=torch.Generator().manual_seed(5))
    w = {k: v.to(F64) for k, v in tensors.items()}
    rms = lambda v, name: plain.rms_norm(v, w[name], 1e-4)
    settings = {"heads": 2, "dim": 16, "rot_dim": 8, "vdim": 24, "kv_rank": 40, "scale": 0.4, "rot": {"dims": 8, "base": 100.0}}
    want = x.to(F64) + 0.3 * rms(plain.latent_attention(rms(x.to(F64), "b.norm1"), w, "b.mix", settings, 1e-4,
                                                        torch.arange(30)), "b.norm1b")
    if with_feed_forward:
        want = want + 0.3 * rms(plain.dense_feed_forward(rms(want, "b.norm2"), w, "b.mlp"), "b.norm2b")
    for ctx, manager, start, n in steps_of_one_request([block.mixer.cache_need()], 30, rt, [30]):
        stream = x.to(DEV).clone()
        pending = block.forward(stream, None, ctx, manager.entries[0])
        assert isinstance(pending, ops.PendingPostNorm)
        close(stream + pending.compute().float(), want, dtype, "the stream after the block")


# ------------------------------------------------------------------ whole models, cut in every way

LENGTHS = [70, 1, 133, 2, 45, 260, 97, 3, 161]
SIZES = [2, 7, 3, 16, 5, 2, 33, 9, 64, 4, 1]


@pytest.fixture(scope="module", params=sorted(ZTINY))
def ztiny(request, tmp_path_factory):
    name = request.param
    return name, make_folder(name, str(tmp_path_factory.mktemp(f"zasesun_{name}"))), ZTINY[name]


CLOSE_CALL = 0.03      # router logits: a bfloat16 run may choose otherwise below this margin


def plain_logits(cfg, weights, tokens):
    """float32 logits of every position, and which positions have a router whose choice between
    the last expert in and the first one out is a close call in some layer: there a bfloat16 run
    may rightly choose the other expert, and its logits are not compared."""
    margins = []
    logits = plain.forward(cfg, weights, tokens, margins=margins).to(torch.float32).numpy()
    close_call = np.zeros(len(tokens), dtype=bool)
    for m in margins:
        close_call |= m.numpy() < CLOSE_CALL
    return logits, close_call


@pytest.mark.parametrize("dtype, sorted_experts", [("float32", False), ("bfloat16", False), ("bfloat16", True)])
def test_every_cutting_matches_plain(ztiny, dtype, sorted_experts, tmp_path, monkeypatch):
    """``sorted_experts``: the routed layers' steps of more than 16 rows sort their rows by expert
    and compute the chosen experts only; else every step computes all experts."""
    name, folder, settings = ztiny
    cfg, weights = load_folder(folder)
    vocab = cfg["vocab"]
    requests = {f"r{i}": tokens_of(vocab, n, seed=200 + i) for i, n in enumerate(LENGTHS)}
    both = {rid: plain_logits(cfg, weights, tokens) for rid, tokens in requests.items()}
    want = {rid: logits for rid, (logits, _) in both.items()}
    unsure = {rid: flags for rid, (_, flags) in both.items()}
    assert sum(int(f.sum()) for f in unsure.values()) < 0.1 * sum(LENGTHS)
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
    cut_decode_tail(b, "r5", requests["r5"], tail=200 if name == "P" else 40)          # long decoding
    section("portions")
    for k, rid in enumerate(("r2", "r4", "r5", "r3")):
        cut_portions(b, rid, requests[rid], SIZES[k:] + SIZES[:k])
    section("mixed")
    cut_mixed(b, requests, SIZES, live=4, seed=6)
    section("end")
    # four live requests, each rounded up to 64 tokens: so few pages that they are used again
    rounded = sorted((-(-n // 64) * 64 for n in LENGTHS), reverse=True)
    monkeypatch.setenv("MRUN_MOE_SORT_MIN_FLOPS", "0" if sorted_experts else "1e30")
    runner = TraceRunner(folder, dtype, str(tmp_path / "out"), sum(rounded[:4]), settings["page_size"], max_requests=4)
    try:
        runner.run(b.steps)
    finally:
        assert runner.close() == 0
    scale = max(float(np.max(np.abs(w))) for w in want.values())
    bound = 2e-5 if dtype == "float32" else 4e-2
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
        if dtype == "bfloat16" and unsure[rid][position]:
            continue
        error = float(np.max(np.abs(got - want[rid][position]))) / scale
        label = [l for l in labels[:-1] if cuts[l] <= index][-1]
        if error > worst.get(label, (0.0,))[0]:
            worst[label] = (error, step, rid, position)
    print(name, dtype, {k: f"{v[0]:.2e}" for k, v in worst.items()})
    for label, (error, step, rid, position) in worst.items():
        assert error <= bound, f"{name}/{dtype}/{label}: error {error:.3e} at step {step}, request {rid}, position {position}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_matches_plain(ztiny, dtype):
    from mrun_b200 import Engine
    name, folder, settings = ztiny
    cfg, weights = load_folder(folder)
    prompts = [tokens_of(cfg["vocab"], n, seed=300 + n) for n in (1, 9, 40, 71, 5)]
    engine = Engine.from_folder(folder, dtype=dtype, page_size=settings["page_size"], context=512,
                                max_batch_tokens=7, max_requests=4)
    results = engine.generate(prompts, max_tokens=10, ignore_eos=True)
    assert bool(engine.executor._graphs) == engine.executor.model.graph_safe
    for prompt, result in zip(prompts, results):
        assert result.finish_reason == "length" and len(result.tokens) == 10
        tokens = list(prompt)
        for n, token in enumerate(result.tokens):
            margins = []
            logits = plain.forward(cfg, weights, tokens, margins=margins)[-1]
            best = int(torch.argmax(logits))
            # bfloat16: both logits may be off by the bound of the logits' test
            margin = 1e-3 if dtype == "float32" else 2 * 4e-2 * float(logits.abs().max())
            unsure = dtype == "bfloat16" and any(float(m[-1]) < CLOSE_CALL for m in margins)
            assert token == best or unsure or float(logits[best] - logits[token]) < margin, \
                f"{name}: output token {n}: engine {token}, plain {best}, behind by {float(logits[best] - logits[token]):.4f}"
            tokens.append(token)
    engine.executor.cache.check_invariants()
    assert not engine.executor.cache.live


def test_command_line_random_then_run(tmp_path):
    """``mrun random`` writes a Zasesun folder from its config.json, ``mrun run`` generates from it."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), os.pardir))
    mrun = os.path.join(root, "bin", "mrun")
    run = lambda *args: subprocess.run([sys.executable, mrun, *args], capture_output=True, text=True, timeout=600)
    (tmp_path / "cfg.json").write_text(json.dumps(ZTINY["P"]["config"]))
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
    assert len(tokens) == 19 + 6 and "Zasesun" in result.stderr
