"""The Loselix design in the engine against the plain implementation (tests/plain/loselix_plain.py): every
mechanism alone, then models of several sizes through the replay program's class (whole, last tokens one by one,
portions down to two tokens, unequal requests side by side in reused pages), special weights where random ones
would hide a fault, and greedy generation through the entry point and its scheduler."""

from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from tests.loselix_util import CONFIGS, PAGE, config, layer, make_weights, sig, soft, stored, twin, write_folder
from tests.plain import loselix_plain as lp
from tests.test_replay_gpu import limits
from tests.util import collect, portions, prefix_then_single, random_tokens, whole

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
LENGTHS = {"la": [70, 45, 100, 33], "lb": [90, 38, 64, 51], "lc": [200, 70, 150, 40], "ld": [61, 40, 83, 35],
           "le": [150, 40, 90, 30]}


def compare(steps, out_dir, vocab, want, dtype, case=None):
    """Every written row against the oracle's.  32-bit holds every position and the greedy token; in bfloat16 one
    position in fifty (or one) may be over the limit by up to half of it."""
    from tests.conftest import record_worst
    got = collect(steps, out_dir, vocab)
    worst, lim_of_worst, total, slightly = 0.0, 0.0, 0, 0
    for rid, rows in got.items():
        lim = limits(dtype, want[rid])
        for pos, row in rows.items():
            total += 1
            w = want[rid][pos]
            diff = (torch.from_numpy(row.copy()) - w).abs().max().item()
            if dtype != "float32" and lim < diff <= 1.5 * lim:
                slightly += 1
                continue
            assert diff <= lim, f"{rid} position {pos}: |diff| {diff:.3e} > {lim:.3e}"
            if diff >= worst:
                worst, lim_of_worst = diff, lim
            if dtype == "float32":
                top2 = w.topk(2).values
                assert int(row.argmax()) == int(w.argmax()) or float(top2[0] - top2[1]) < 1e-4
    assert slightly <= max(1, 0.02 * total), f"{slightly} of {total} positions are over the limit"
    if case is not None:
        record_worst(case, dtype, worst, lim_of_worst)
    return got


@pytest.fixture(scope="module", params=sorted(CONFIGS))
def setup(request, tmp_path_factory):
    tag = request.param
    c = CONFIGS[tag]
    weights = make_weights(c, seed=5)
    folder = write_folder(tmp_path_factory.mktemp(f"loselix_{tag}"), c, weights)
    w = stored(weights)
    seqs = {f"r{i}": random_tokens(n, c["vocab"], seed=20 + i) for i, n in enumerate(LENGTHS[tag])}
    want = {rid: lp.forward(c, w, t).to(torch.float32) for rid, t in seqs.items()}
    assert all(v.abs().max() > 1.0 for v in want.values())     # logits of order one, not a flat model
    return tag, folder, seqs, want


def replay(folder, tag, dtype, steps, out_dir, max_tokens, **switches):
    from jax_vllm_b200.engine.replay import Replayer
    rep = Replayer(folder, dtype, out_dir, max_tokens=max_tokens, page_size=PAGE[tag], **switches)
    rep.run_stream(json.dumps(s) for s in steps)
    rep.cache.check()
    assert not rep.cache.live
    return rep


# ------------------------------------------------------------------ mechanisms alone
def scrambled_pages(ctx_new, P, n_pages, g):
    """A block table over pages in a random order for entries of (cached, new) tokens."""
    width = max(-(-(c + q) // P) for c, q in ctx_new)
    table = torch.full((len(ctx_new), width), -1, dtype=torch.int32)
    free = torch.randperm(n_pages, generator=g).tolist()
    for e, (c, q) in enumerate(ctx_new):
        for i in range(-(-(c + q) // P)):
            table[e, i] = free.pop()
    return table


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", ["whole_norm_temperature_values_from_keys", "rotation_of_a_part", "plain"])
def test_prepare_alone(dtype, case):
    """Queries, and keys and values in their pages, at positions far from 0 and next to the edges of the
    temperature's steps, on pages given in a scrambled order; untouched places stay untouched."""
    from jax_vllm_b200 import ops
    g = torch.Generator().manual_seed(7)
    Hq, Hk, D = 6, 2, 20
    normed = case.startswith("whole")
    Hv, DV = (Hk, D) if normed else (1, 12)
    rot = 8 if case == "rotation_of_a_part" else 0
    coef, every = (0.4, 16) if normed else (0.0, 0)
    P, base, eps = 4, 3e4, 1e-5
    positions = torch.tensor([0, 14, 15, 16, 31, 32, 1001, 1002, 30000], dtype=torch.int32)
    entry = torch.tensor([0, 0, 0, 0, 0, 0, 1, 1, 2], dtype=torch.int32)
    n = positions.numel()
    k_off, v_off = Hq * D + 3, (-1 if normed else Hq * D + 3 + Hk * D + 5)
    row = torch.randn((n, Hq * D + Hk * D + Hv * DV + 11), generator=g).to(dtype)
    qw = (1 + 0.1 * torch.randn(Hq * D, generator=g)).to(torch.bfloat16) if normed else None
    kw = (1 + 0.1 * torch.randn(Hk * D, generator=g)).to(torch.bfloat16) if normed else None
    inv_freq = (base ** (-torch.arange(0, rot, 2, dtype=torch.float64) / rot)).float() if rot else None
    table = torch.full((3, 30000 // P + 1), -1, dtype=torch.int32)
    pages = torch.randperm(16, generator=g).tolist()
    where = []
    for t in range(n):
        e, p = int(entry[t]), int(positions[t])
        if table[e, p // P] < 0:
            table[e, p // P] = pages.pop()
        where.append((int(table[e, p // P]), p % P))
    kc = torch.full((16, P, Hk, D), float("nan"), dtype=dtype).cuda()
    vc = torch.full((16, P, Hv, DV), float("nan"), dtype=dtype).cuda()
    q = torch.zeros((n, Hq * D), dtype=dtype).cuda()
    ops.attn_prepare(row.cuda(), 0, k_off, v_off, q, positions.cuda(), entry.cuda(), table.cuda(),
                     None if inv_freq is None else inv_freq.cuda(), None if qw is None else qw.cuda(),
                     None if kw is None else kw.cuda(), eps, coef, every, kc, vc, Hq, Hk, Hv, D, DV)
    ops.check_status()
    r64 = row.double()
    q_raw, k_raw = r64[:, :Hq * D], r64[:, k_off:k_off + Hk * D]
    v_want = k_raw if normed else r64[:, v_off:v_off + Hv * DV]
    q_want, k_want = q_raw, k_raw
    if normed:
        q_want, k_want = lp.rms_norm(q_raw, qw.double(), eps), lp.rms_norm(k_raw, kw.double(), eps)
        q_want = q_want * lp.query_temperature(positions, coef, every)[:, None]
    q_want, k_want = q_want.view(n, Hq, D), k_want.view(n, Hk, D)
    if rot:
        q_want, k_want = lp.rotate_first(q_want, positions, rot, base), lp.rotate_first(k_want, positions, rot, base)
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    far = positions >= 2000                                   # 32-bit angles at position 30000 carry about 1e-3
    gq, gk, gv = q.cpu().double().view(n, Hq, D), kc.cpu().double(), vc.cpu().double()
    for t, (page, slot) in enumerate(where):
        t_tol = tol * (40 if (far[t] and rot) else 1)
        assert (gq[t] - q_want[t]).abs().max() < t_tol
        assert (gk[page, slot] - k_want[t]).abs().max() < t_tol
        assert (gv[page, slot].flatten() - v_want[t]).abs().max() < 1e-6 * (1 if dtype == torch.float32 else 1e4)
    written = torch.zeros((16, P), dtype=torch.bool)
    for page, slot in where:
        written[page, slot] = True
    assert torch.isnan(gk[~written]).all() and torch.isnan(gv[~written]).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_finish_alone(dtype):
    from jax_vllm_b200 import ops
    g = torch.Generator().manual_seed(8)
    n, H, E = 9, 3, 20
    a = torch.randn((n, 2 * H * E), generator=g)
    wide = torch.randn((n, 7 + H * E + H), generator=g).to(dtype)
    tol = 2e-6 if dtype == torch.float32 else 2e-2
    # two maps: a1 - lam * a2, unit norm over the head, times a constant; written into a column range
    out = torch.full((n, H * E + 5), float("nan"), dtype=dtype).cuda()
    ops.attn_finish(a.cuda(), out[:, 5:], H, E, maps=2, lam=0.7, unit_norm_eps=1e-5, post=0.6)
    a64 = a.double().view(n, 2, H, E)
    want = lp.unit_rms(a64[:, 0] - 0.7 * a64[:, 1], 1e-5) * 0.6
    assert (out[:, 5:].cpu().double().view(n, H, E) - want).abs().max() < tol and torch.isnan(out[:, :5]).all()
    # one map with a gate per head, then per element, read from a column range of a wider tensor
    one = a[:, :H * E].to(dtype)
    for cols, shape in ((slice(7 + H * E, 7 + H * E + H), (n, H, 1)), (slice(7, 7 + H * E), (n, H, E))):
        out = torch.empty((n, H * E), dtype=dtype).cuda()
        ops.attn_finish(one.cuda(), out, H, E, gate=wide.cuda()[:, cols])
        want = one.double().view(n, H, E) * torch.sigmoid(wide[:, cols].double().reshape(shape))
        assert (out.cpu().double().view(n, H, E) - want).abs().max() < tol


def test_small_kernels_alone():
    from jax_vllm_b200 import ops
    g = torch.Generator().manual_seed(9)
    z = torch.randn((5, 37), generator=g)
    wide = torch.zeros((5, 50)).cuda()
    ops.unary_act(z.cuda()[:, 3:30], "relu2", wide[:, 11:38])
    assert torch.equal(wide[:, 11:38].cpu(), torch.relu(z[:, 3:30]) ** 2) and (wide[:, :11] == 0).all() and (wide[:, 38:] == 0).all()
    table = torch.randn((20, 24), generator=g).to(torch.bfloat16)
    ids = torch.tensor([3, 19, 0, 3], dtype=torch.int32)
    h = torch.randn((4, 24), generator=g)
    hd = h.cuda()
    ops.embed_gather(table.cuda(), ids.cuda(), out=hd, accumulate=True)
    assert torch.equal(hd.cpu(), h + table[ids.long()].float())


ATTENTION_CASES = {
    # name: (query heads, key heads, value heads, key size, value size, cap, sigmoid)
    "twin_like_capped": (8, 4, 2, 48, 96, 6.0, False),
    "sigmoid_biased": (6, 2, 2, 32, 32, 0.0, True),
    "values_wider_no_group": (3, 3, 3, 16, 64, 0.0, False),
    "sigmoid_capped_long_keys": (4, 1, 1, 160, 16, 3.0, True),
}


@pytest.mark.parametrize("kernel", ["simt32", "simt16", "mma16"])
@pytest.mark.parametrize("name", sorted(ATTENTION_CASES))
def test_attention_kernels_alone(name, kernel):
    """The CUDA-core kernel (32-bit, and on 16-bit rows) and the tensor-core kernel compiled per pair of sizes
    against the plain functions: a prompt portion over several tiles with earlier context, a short prompt from
    position 0, a single token split along its keys; pages in a scrambled order, unowned places NaN."""
    from jax_vllm_b200 import ops
    Hq, Hk, Hv, D, E, cap, sigmoid = ATTENTION_CASES[name]
    dtype = torch.float32 if kernel == "simt32" else torch.bfloat16
    g = torch.Generator().manual_seed(Hq * D + E)
    P, n_pages, scale = 8, 64, D ** -0.5
    ctx_new = [(37, 45), (0, 3), (130, 1)]
    table = scrambled_pages(ctx_new, P, n_pages, g)
    kc = torch.full((n_pages, P, Hk, D), float("nan"), dtype=dtype)
    vc = torch.full((n_pages, P, Hv, E), float("nan"), dtype=dtype)
    ks, vs, qs = [], [], []
    for e, (c, q) in enumerate(ctx_new):
        k = (torch.randn((c + q, Hk, D), generator=g) * 1.5).to(dtype)
        v = torch.randn((c + q, Hv, E), generator=g).to(dtype)
        for j in range(c + q):
            kc[table[e, j // P], j % P], vc[table[e, j // P], j % P] = k[j], v[j]
        ks.append(k.double()); vs.append(v.double())
        qs.append((torch.randn((q, Hq, D), generator=g) * 1.5).to(dtype))
    bias = (torch.randn(Hq, generator=g) - 1.0) if sigmoid else None
    n = sum(q for _, q in ctx_new)
    q_all = torch.cat(qs).reshape(n, Hq * D).cuda()
    cu = torch.tensor([0, 45, 48, 49], dtype=torch.int32).cuda()
    start = torch.tensor([c for c, _ in ctx_new], dtype=torch.int32).cuda()
    out = torch.full((n, Hq * E), float("nan"), dtype=torch.float32).cuda()       # float output from 16-bit rows too
    extra = dict(score_cap=cap, sigmoid=sigmoid, bias=None if bias is None else bias.cuda())
    common = (kc.cuda(), vc.cuda(), table.cuda(), cu, start)
    if kernel == "mma16":
        assert ops.attn_general_mma_supports(dtype, D, E)
        tpt = ops.attn_general_mma_tokens_per_tile(Hq, Hk)
        run = lambda work, **split: ops.attn_general_mma(q_all, Hq * D, out, *common, work, work.shape[0], Hq, Hk, scale, **split, **extra)
    else:
        tpt = ops.attn_simt_tokens_per_tile(Hq, Hk)
        run = lambda work, **split: ops.attn_simt(q_all, Hq * D, out, *common, work, work.shape[0], Hq, Hk, D, 0, scale,
                                                  v_dim=E, **split, **extra)
    tiles = [(0, t) for t in range(0, 45, tpt)] + [(1, t) for t in range(0, 3, tpt)]
    run(torch.tensor(tiles, dtype=torch.int32).cuda())
    run(torch.tensor([(2, 0)], dtype=torch.int32).cuda(), split_size=64, n_splits=3)
    ops.check_status()
    got = out.cpu().double().view(n, Hq, E)
    at = 0
    for e, (c, q) in enumerate(ctx_new):
        T = c + q
        q_full = torch.zeros((T, Hq, D), dtype=torch.float64)
        q_full[c:] = qs[e].double()
        want = torch.zeros((T, Hq, E), dtype=torch.float64)
        per = Hk // Hv                      # key heads per value head: key head g reads value head g % Hv
        for m in range(per):
            qh = slice(m * Hq // per, (m + 1) * Hq // per)
            s = lp.causal_scores(q_full[:, qh], ks[e][:, m * Hv:(m + 1) * Hv], scale)
            if cap:
                s = lp.tanh_cap(s, cap)
            want[:, qh] = lp.sigmoid_attend(s, bias.double()[qh], vs[e]) if sigmoid else lp.softmax_attend(s, vs[e])
        tol = 2e-5 if kernel == "simt32" else 2.5e-2
        assert (got[at:at + q] - want[c:]).abs().max() < tol * max(1.0, want[c:].abs().max().item())
        at += q


@pytest.mark.parametrize("Hq,Hk", [(4, 2), (3, 3), (8, 1)])
def test_sigmoid_weights_on_the_tcgen05_kernel(Hq, Hk):
    """Whole 128-row tiles of a prompt portion with sigmoid weights and a bias per head, heads of 128, earlier context
    in the cache, a last tile that is not full, and an entry that is exactly one tile."""
    from jax_vllm_b200 import ops
    D, P, n_pages, scale = 128, 16, 40, 128 ** -0.5
    tpt = ops.attn_tcgen05_tokens_per_tile(Hq, Hk)
    ctx_new = [(100, 2 * tpt + 22), (0, tpt)]
    g = torch.Generator().manual_seed(Hq)
    table = scrambled_pages(ctx_new, P, n_pages, g)
    kc = torch.full((n_pages, P, Hk, D), float("nan"), dtype=torch.bfloat16)
    vc = torch.full((n_pages, P, Hk, D), float("nan"), dtype=torch.bfloat16)
    ks, vs, qs = [], [], []
    for e, (c, q) in enumerate(ctx_new):
        k = (torch.randn((c + q, Hk, D), generator=g) * 1.5).to(torch.bfloat16)
        v = torch.randn((c + q, Hk, D), generator=g).to(torch.bfloat16)
        for j in range(c + q):
            kc[table[e, j // P], j % P], vc[table[e, j // P], j % P] = k[j], v[j]
        ks.append(k.double()); vs.append(v.double())
        qs.append((torch.randn((q, Hq, D), generator=g) * 1.5).to(torch.bfloat16))
    bias = torch.randn(Hq, generator=g) - 2.0
    n = sum(q for _, q in ctx_new)
    q_all = torch.cat(qs).reshape(n, Hq * D).cuda()
    cu = torch.tensor([0, ctx_new[0][1], n], dtype=torch.int32).cuda()
    start = torch.tensor([c for c, _ in ctx_new], dtype=torch.int32).cuda()
    out = torch.full((n, Hq * D), float("nan"), dtype=torch.bfloat16).cuda()
    tiles = [(e, t) for e, (_, q) in enumerate(ctx_new) for t in range(0, q, tpt)]
    ops.attn_tcgen05(q_all, Hq * D, out, kc.cuda(), vc.cuda(), table.cuda(), cu, start,
                     torch.tensor(tiles, dtype=torch.int32).cuda(), len(tiles), Hq, Hk, D, scale, sigmoid=True, bias=bias.cuda())
    ops.check_status()
    got = out.cpu().double().view(n, Hq, D)
    at = 0
    for e, (c, q) in enumerate(ctx_new):
        q_full = torch.zeros((c + q, Hq, D), dtype=torch.float64)
        q_full[c:] = qs[e].double()
        want = lp.sigmoid_attend(lp.causal_scores(q_full, ks[e], scale), bias.double(), vs[e])[c:]
        assert (got[at:at + q] - want).abs().max() < 2.5e-2 * max(1.0, want.abs().max().item())
        at += q


def test_a_size_pair_outside_the_tensor_core_kernel_is_told():
    from jax_vllm_b200 import ops
    assert not ops.attn_general_mma_supports(torch.bfloat16, 24, 32)
    assert not ops.attn_general_mma_supports(torch.float32, 32, 32)
    assert ops.attn_general_mma_supports(torch.bfloat16, 96, 96)


# ------------------------------------------------- whole models through the replay class
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompt(setup, dtype, tmp_path):
    tag, folder, seqs, want = setup
    steps = whole("r0", seqs["r0"])
    replay(folder, tag, dtype, steps, tmp_path, max_tokens=256)
    compare(steps, tmp_path, CONFIGS[tag]["vocab"], want, dtype, case=f"loselix {tag}, whole")


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_last_tokens_one_by_one(setup, dtype, graphs, tmp_path):
    tag, folder, seqs, want = setup
    steps = prefix_then_single("r1", seqs["r1"], tail=20)
    rep = replay(folder, tag, dtype, steps, tmp_path, max_tokens=128, cuda_graphs=graphs)
    compare(steps, tmp_path, CONFIGS[tag]["vocab"], want, dtype, case=f"loselix {tag}, decoded")
    assert (rep.runner.graph_replays > 0) == graphs


@pytest.mark.parametrize("sizes", [(2,), (5, 1, 2, 19), (33, 3)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions(setup, dtype, sizes, tmp_path):
    tag, folder, seqs, want = setup
    steps = portions("r2", seqs["r2"], sizes)
    replay(folder, tag, dtype, steps, tmp_path, max_tokens=192)
    compare(steps, tmp_path, CONFIGS[tag]["vocab"], want, dtype, case=f"loselix {tag}, portions")


def mixed_trace(seqs):
    """Four requests, never more than three live: portions of some beside single tokens of others; r3 starts only
    after r1 has ended, in the pages and the slot that r1 gave back; r1 is left out of a step and goes on later."""
    plan = [{"r0": 9, "r1": 2}, {"r0": 1, "r1": 17, "r2": 30}, {"r0": 30, "r2": 1}, {"r0": 1, "r1": 1, "r2": 2},
            {"r0": 1, "r1": 999, "r2": 1}, {"r0": 999, "r2": 40, "r3": 3}, {"r2": 999, "r3": 1}, {"r3": 999}]
    fed = {r: 0 for r in seqs}
    steps = []
    for k, row in enumerate(plan):
        entries = []
        for rid, n in row.items():
            part = seqs[rid][fed[rid]:fed[rid] + n]
            if part:
                entries.append({"id": rid, "tokens": part, "want": list(range(len(part)))})
                fed[rid] += len(part)
        steps.append({"step": k, "entries": entries, "end": [e["id"] for e in entries if fed[e["id"]] == len(seqs[e["id"]])]})
    assert all(fed[r] == len(seqs[r]) for r in seqs)
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_requests_side_by_side_in_reused_pages(setup, dtype, tmp_path):
    tag, folder, seqs, want = setup
    steps = mixed_trace(seqs)
    P = PAGE[tag]
    live3 = sum(sorted(-(-len(s) // P) * P for s in seqs.values())[-3:])
    rep = replay(folder, tag, dtype, steps, tmp_path, max_tokens=live3)
    compare(steps, tmp_path, CONFIGS[tag]["vocab"], want, dtype, case=f"loselix {tag}, side by side")
    assert sum(m["pages_allocated"] for m in rep.records) > rep.cache.num_pages * len(rep.cache.groups)   # pages came back and went out again


def test_schedules_agree_with_each_other_in_32_bit(setup, tmp_path):
    """A position's logits do not depend on the cut, the batch or the pages beyond rounding."""
    tag, folder, seqs, _ = setup
    V = CONFIGS[tag]["vocab"]
    a = whole("r0", seqs["r0"])
    b = portions("r0", seqs["r0"], (5, 1, 2, 19))
    c = mixed_trace(seqs)
    replay(folder, tag, "float32", a, tmp_path / "a", 256)
    replay(folder, tag, "float32", b, tmp_path / "b", 256)
    replay(folder, tag, "float32", c, tmp_path / "c", 512)
    ga, gb, gc = (collect(s, tmp_path / d, V)["r0"] for s, d in ((a, "a"), (b, "b"), (c, "c")))
    for pos in ga:
        assert abs(ga[pos] - gb[pos]).max() < 3e-5 and abs(ga[pos] - gc[pos]).max() < 3e-5


def test_packed_products_equal_the_parts_run_one_by_one(tmp_path):
    """The parallel block's two products (stacked inputs, outputs joined along k) against the same layers with
    every part running its own products and the branches added one after the other."""
    from jax_vllm_b200.parts.block import ParallelBlock
    c = CONFIGS["lb"]
    weights = make_weights(c, seed=6)
    folder = write_folder(tmp_path / "model", c, weights)
    tokens = random_tokens(60, c["vocab"], seed=3)
    steps = portions("r", tokens, (25, 1, 7))
    replay(folder, "lb", "float32", steps, tmp_path / "packed", 64)
    bind = ParallelBlock.bind

    def unpacked(self, tensors):
        bind(self, tensors)
        self.w_in = self.w_out = None
    ParallelBlock.bind = unpacked
    try:
        replay(folder, "lb", "float32", steps, tmp_path / "apart", 64)
    finally:
        ParallelBlock.bind = bind
    a, b = (collect(steps, tmp_path / d, c["vocab"])["r"] for d in ("packed", "apart"))
    want = lp.forward(c, stored(weights), tokens).float()
    for pos in a:
        assert abs(a[pos] - b[pos]).max() < 3e-5 and abs(torch.from_numpy(b[pos].copy()) - want[pos]).max() < 1e-4


def test_trace_run_program(tmp_path):
    """bin/trace_run as a program on a Loselix folder: stdin steps, `done <step>` lines, files on disk, exit 0."""
    c = CONFIGS["la"]
    weights = make_weights(c, seed=9)
    folder = write_folder(tmp_path / "model", c, weights)
    seqs = {f"r{i}": random_tokens(n, c["vocab"], seed=40 + i) for i, n in enumerate([40, 21, 33, 12])}
    want = {rid: lp.forward(c, stored(weights), t).to(torch.float32) for rid, t in seqs.items()}
    steps = mixed_trace(seqs)
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32",
                           "--out", str(tmp_path / "out"), "--max-tokens", "192"],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
                          env=dict(os.environ), timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == [w for s in steps for w in ("done", str(s["step"]))]
    compare(steps, tmp_path / "out", c["vocab"], want, "float32")


# ------------------------------------------------------- weights that make a fault show
def special(tmp_path, c, weights, tokens, dtype, sizes=None, page=16, tail=0):
    from jax_vllm_b200.engine.replay import Replayer
    folder = write_folder(tmp_path / "model", c, weights)
    if tail:
        steps = prefix_then_single("r", tokens, tail=tail)
    else:
        steps = whole("r", tokens) if sizes is None else portions("r", tokens, sizes)
    out = tmp_path / f"out_{dtype}_{sizes}_{tail}"
    rep = Replayer(folder, dtype, out, max_tokens=-(-len(tokens) // 64) * 64, page_size=page)
    rep.run_stream(json.dumps(s) for s in steps)
    return steps, out


FAR_LAYERS = {"soft": soft(2, 1, 16, 16, rot=4, scale=0.5), "sigmoid": sig(2, 1, 32, every=64, scale=0.25),
              "twin": twin(2, 1, 24, 40, rot=6, softcap=40.0, diff=0.3, scale=0.5)}


def far_key_model(kind):
    """One layer without a feed-forward in which the last token (2) asks for token 1 wherever that stands, and for
    nothing else.  Token 1's embedding is the first unit vector, token 2's is minus that, and no other token has
    a first component.  In every block of the key matrix (a map of a head) the first column is a vector b that is
    zero on the rotated elements, and the other columns are made orthogonal to b: the key of token 1 is a multiple
    of b, every other key is orthogonal to it wherever it stands.  The first column of every query head's matrix
    is minus three times that of its key head: q(token 2) points along k(token 1), away from its own key, and
    scores 0 on all others."""
    c = config(50, 64, [layer(FAR_LAYERS[kind], None)], eps=1e-5)
    w = make_weights(c, seed=11)
    mx = c["layers"][0]["mixer"]
    H, G, D = mx["heads"], mx["kv_heads"], mx["dim"]
    maps = 2 if kind == "twin" else 1
    rot = mx.get("rot", {}).get("dims", 0)
    w["embed"][:, 0] = 0.0
    w["embed"][1] = 0.0
    w["embed"][1, 0] = 4.0
    w["embed"][2] = -w["embed"][1]
    w["l0.norm1"][0] = 1.0
    wk = w["l0.mix.k"].view(G * maps, D, 64).clone()
    g = torch.Generator().manual_seed(12)
    for blk in range(G * maps):
        b = torch.randn(D, generator=g)
        b[:rot] = 0.0
        b = b / b.norm() * (0.29 if kind != "sigmoid" else 1.0)          # scale * 3 * 64 * |b|^2 is about 8
        rest = wk[blk][:, 1:]
        wk[blk][:, 1:] = rest - b[:, None] * (b @ rest)[None, :] / (b @ b)
        wk[blk][:, 0] = b
    w["l0.mix.k"] = wk.reshape(G * maps * D, 64).contiguous()
    # only tokens 1 and 2 have a first component: every other token's query stays an ordinary random one
    w["l0.mix.q"][:, 0] = (-3.0 * wk.view(G, maps * D, 64).repeat_interleave(H // G, dim=0)).reshape(H * maps * D, 64)[:, 0]
    if kind == "sigmoid":
        w["l0.mix.q.norm"][:] = 1.0
        w["l0.mix.k.norm"][:] = 1.0
        w["l0.mix.pb"][:] = -6.0
    return c, w


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("far", [0, 1, 15, 16, 17, 255, 256])
@pytest.mark.parametrize("kind", sorted(FAR_LAYERS))
def test_one_far_key_among_hundreds(kind, far, dtype, tmp_path):
    """Token 1 stands at position `far` only (the first tokens, a page's last and first places) among 600 tokens.
    The plain implementation's last logits change greatly when it is taken away; the engine's must equal the
    result with it: whole, in portions and decoded."""
    c, w = far_key_model(kind)
    w64 = stored(w)
    tokens = [3 + (i * 7) % 40 for i in range(600)]
    tokens[far], tokens[-1] = 1, 2
    with_key = lp.forward(c, w64, tokens).to(torch.float32)
    without = list(tokens)
    without[far] = 4
    gone = lp.forward(c, w64, without).to(torch.float32)
    assert (with_key[-1] - gone[-1]).abs().max() > 0.5                   # the far key decides the last logits
    for sizes, tail in ((None, 0), ((100, 3, 2), 0), (None, 9)):
        steps, out = special(tmp_path, c, w, tokens, dtype, sizes=sizes, tail=tail)
        compare(steps, out, 50, {"r": with_key}, dtype, case=f"loselix one far key ({kind})")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_temperatures_steps_and_the_first_tokens(dtype, tmp_path):
    """A query temperature that changes every 3 positions with a large coefficient, decoded across several of its
    steps and cut into portions of two tokens: a position that is one off shows from the first tokens on."""
    c = config(64, 32, [layer(sig(2, 2, 16, coef=2.5, every=3, scale=0.6), 24)], eps=1e-6, loop=(0, 1, 3))
    w = make_weights(c, seed=17)
    tokens = random_tokens(40, 64, seed=18)
    want = lp.forward(c, stored(w), tokens).to(torch.float32)
    shifted = {**c, "layers": [layer(sig(2, 2, 16, coef=2.5, every=4, scale=0.6), 24)]}
    assert (lp.forward(shifted, stored(w), tokens).float() - want)[2:8].abs().max() > 0.05    # the steps' places matter early
    for sizes, tail in ((None, 0), ((2,), 0), (None, 30)):
        steps, out = special(tmp_path, c, w, tokens, dtype, sizes=sizes, page=4, tail=tail)
        compare(steps, out, 64, {"r": want}, dtype, case="loselix temperature steps")


# ----------------------------------------------------------- generation, scheduler, entry point
def plain_greedy(c, w, prompt, n):
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(lp.forward(c, w, seq)[-1].argmax()))
    return seq[len(prompt):]


def test_greedy_generation_through_the_entry_point(tmp_path):
    """make_driver + generate: the scheduler's portions, decode steps from captured graphs, sampling."""
    from jax_vllm_b200 import SamplingParams, generate, load_from_path, make_driver
    c = CONFIGS["la"]
    weights = make_weights(c, seed=21)
    folder = write_folder(tmp_path / "model", c, weights)
    model = load_from_path(folder, dtype="fp32")
    d = make_driver(model, max_num_seqs=3, max_model_len=96, block_size=16, max_tokens_per_step=16)
    prompts = [random_tokens(n, c["vocab"], seed=50 + n) for n in (21, 5, 40)]
    got = generate(d, prompts, SamplingParams(max_new_tokens=40))
    assert got == [plain_greedy(c, stored(weights), p, 40) for p in prompts]     # long decoding: 40 tokens each
    assert d.runner.graph_replays > 0
    d.cache.check()


def test_random_arrivals_with_few_pages(tmp_path):
    """Requests arrive at random steps into a pool too small for them: the youngest is preempted and run again,
    pages and slots come back and are used again; greedy tokens depend on none of it."""
    import random
    from jax_vllm_b200 import SamplingParams, add_request, has_work, load_from_path, make_driver, step
    c = CONFIGS["lb"]
    weights = make_weights(c, seed=22)
    folder = write_folder(tmp_path / "model", c, weights)
    rng = random.Random(1)
    model = load_from_path(folder, dtype="fp32")
    d = make_driver(model, max_num_seqs=3, max_model_len=64, block_size=8, num_blocks=9, max_tokens_per_step=24)
    prompts = [random_tokens(rng.randrange(1, 30), c["vocab"], seed=100 + i) for i in range(8)]
    new_tokens = [rng.randrange(6, 27) for _ in prompts]
    waiting, ids = list(range(len(prompts))), {}
    while waiting or has_work(d):
        if waiting and (rng.random() < 0.4 or not has_work(d)):
            i = waiting.pop(0)
            ids[i] = add_request(d, prompts[i], SamplingParams(max_new_tokens=new_tokens[i]))
        step(d)
        d.cache.check()
    assert not d.cache.live and all(g.pool.num_free == 9 for g in d.cache.groups)
    assert d.stats.preemptions > 0
    w = stored(weights)
    for i, prompt in enumerate(prompts):
        assert d.requests[ids[i]].output_ids == plain_greedy(c, w, prompt, new_tokens[i]), f"request {i}"


def test_command_line(tmp_path):
    """cli.py as a user runs it on a Loselix folder: prompts as token ids, 32-bit; the printed ids are the plain
    implementation's greedy tokens (prefix reuse is on by default: the second prompt repeats the first one's start)."""
    c = CONFIGS["le"]
    weights = make_weights(c, seed=23)
    folder = write_folder(tmp_path / "model", c, weights)
    prompts = [random_tokens(37, c["vocab"], seed=60), random_tokens(37, c["vocab"], seed=60)[:33] + [5, 6], [9]]
    cmd = [sys.executable, str(ROOT / "cli.py"), "--model-path", str(folder), "--dtype", "fp32", "--max-tokens", "7",
           "--max-model-len", "128", "--block-size", "32", "--no-prewarm"]
    for p in prompts:
        cmd += ["--prompt-ids", ",".join(map(str, p))]
    proc = subprocess.run(cmd, capture_output=True, text=True, env=dict(os.environ), timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    got = [json.loads(line)["output_ids"] for line in proc.stdout.splitlines() if line.startswith("{")]
    assert got == [plain_greedy(c, stored(weights), p, 7) for p in prompts]


def test_sampled_tokens_depend_on_the_seed_not_on_the_batch(tmp_path):
    """Temperature sampling through the entry point: a request's tokens depend on its seed, not on what runs beside it."""
    from jax_vllm_b200 import SamplingParams, generate, load_from_path, make_driver
    c = CONFIGS["ld"]
    folder = write_folder(tmp_path / "model", c, make_weights(c, seed=24))
    model = load_from_path(folder, dtype="fp32")
    prompts = [random_tokens(n, c["vocab"], seed=70 + n) for n in (11, 3, 25)]
    sp = [SamplingParams(max_new_tokens=12, temperature=0.8, seed=100 + i) for i in range(3)]
    together = generate(make_driver(model, max_num_seqs=3, max_model_len=64, block_size=4), prompts, sp)
    alone = [generate(make_driver(model, max_num_seqs=1, max_model_len=64, block_size=4), [p], [s])[0]
             for p, s in zip(prompts, sp)]
    assert together == alone
    other = generate(make_driver(model, max_num_seqs=1, max_model_len=64, block_size=4), [prompts[0]],
                     [SamplingParams(max_new_tokens=12, temperature=0.8, seed=999)])[0]
    assert other != alone[0]


def random_configuration(seed):
    """A configuration drawn at random: every size, the order of the layers, the loop and which options are there."""
    import random
    rng = random.Random(seed)
    width = rng.choice([40, 50, 64, 72, 100, 128, 136])
    sizes = [6, 8, 16, 20, 32, 48, 64, 80, 96, 128]
    layers = []
    for _ in range(rng.randint(1, 5)):
        kv = rng.choice([1, 2, 3])
        heads = kv * rng.choice([1, 2, 4])
        dim, vdim = rng.choice(sizes), rng.choice(sizes)
        kind = rng.choice(["soft", "sigmoid", "twin"])
        rot = rng.choice([None, 2 * rng.randint(1, dim // 2)])
        if kind == "soft":
            mixer = soft(heads, kv, dim, rng.choice([dim, vdim]), rot=rot, base=rng.choice([1e4, 5e5]))
        elif kind == "sigmoid":
            mixer = sig(heads, kv, dim, coef=rng.uniform(0.1, 0.6), every=rng.choice([0, 3, 16, 50]))
        else:
            mixer = twin(heads, kv, dim, vdim, rot=rot, softcap=rng.choice([0.0, 8.0, 50.0]), diff=rng.uniform(0.1, 0.5))
        layers.append(layer(mixer, rng.choice([None, 24, 56, 100])))
    n = len(layers)
    loop = None
    if rng.random() < 0.7:
        a = rng.randrange(n)
        loop = (a, rng.randint(a + 1, n), rng.randint(1, 3))
    return config(rng.choice([97, 160, 333]), width, layers, eps=rng.choice([1e-6, 1e-5]), loop=loop)


@pytest.mark.parametrize("seed", range(10))
def test_configurations_drawn_at_random(seed, tmp_path):
    """Sizes, layer orders, loops and options that nobody chose: portions of changing size, then single tokens, two
    requests side by side, in both precisions."""
    from jax_vllm_b200.engine.replay import Replayer
    c = random_configuration(seed)
    weights = make_weights(c, seed=100 + seed)
    folder = write_folder(tmp_path / "model", c, weights)
    seqs = {"a": random_tokens(75, c["vocab"], seed=seed), "b": random_tokens(41, c["vocab"], seed=50 + seed)}
    want = {rid: lp.forward(c, stored(weights), t).to(torch.float32) for rid, t in seqs.items()}
    plan = [{"a": 20}, {"a": 2, "b": 30}, {"a": 33, "b": 1}] + [{"a": 1, "b": 1}] * 10 + [{"a": 999}]
    fed = {r: 0 for r in seqs}
    steps = []
    for k, row in enumerate(plan):
        entries = []
        for rid, n in row.items():
            part = seqs[rid][fed[rid]:fed[rid] + n]
            if part:
                entries.append({"id": rid, "tokens": part, "want": list(range(len(part)))})
                fed[rid] += len(part)
        steps.append({"step": k, "entries": entries, "end": [e["id"] for e in entries if fed[e["id"]] == len(seqs[e["id"]])]})
    for dtype in ("float32", "bfloat16"):
        rep = Replayer(folder, dtype, tmp_path / dtype, max_tokens=128, page_size=16)
        rep.run_stream(json.dumps(s) for s in steps)
        rep.cache.check()
        compare(steps, tmp_path / dtype, c["vocab"], want, dtype, case="loselix drawn at random")
