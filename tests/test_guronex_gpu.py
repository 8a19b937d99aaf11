"""The Guronex design in the engine against the plain implementation (tests/plain/guronex_plain.py): every
mechanism alone, then models of several sizes through the replay program's class (whole, last tokens one by one,
portions down to two tokens, unequal requests side by side in reused pages), special weights where random ones
would hide a fault, and greedy generation through the entry point and its scheduler."""

from __future__ import annotations

import copy
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from tests.guronex_util import CONFIGS, PAGE, config, layer, make_weights, mixer, moe, write_folder
from tests.plain import guronex_plain as gp
from tests.test_replay_gpu import limits
from tests.util import portions, prefix_then_single, random_tokens, whole

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
LENGTHS = {"ga": [70, 45, 100, 33], "gb": [90, 38, 64, 51], "gc": [200, 70, 150, 40], "gd": [61, 40, 83, 35],
           "ge": [80, 37, 50, 20], "gf": [150, 40, 90, 30], "gg": [150, 40, 90, 30], "gh": [70, 45, 100, 33]}


CLOSE_CALL = 0.1       # a difference of router logits below which bfloat16 may choose another expert
EXCUSED = 0.25         # share of the positions that may differ for that reason (where the choice cannot be followed)


def oracle(c, w, tokens):
    """(logits, positions whose routing is a close call in some layer)."""
    margins = []
    logits = gp.forward(c, w, tokens, margins=margins).to(torch.float32)
    close = set()
    for m in margins:
        close.update(torch.nonzero(m < CLOSE_CALL).flatten().tolist())
    return logits, close


def compare(steps, out_dir, vocab, want, dtype, case=None, close=None, floor=None):
    """Every written row against the oracle's; 32-bit holds every position.  In bfloat16 a token whose choice of
    experts hangs on a small difference of router logits (`close`: request -> positions where the oracle finds
    one) may choose otherwise, and what comes after it attends to the changed token: a position over the limit is
    excused only if such a token stands at or before it, and no more than EXCUSED of all positions are.  `floor`
    (request -> per position) is what rounding alone does to the plain implementation's logits (its own 32-bit
    run where a case is badly conditioned by design; its run with the branches' inputs rounded to 16 bits for
    bfloat16); the limit is at least 3 times it.  In bfloat16 one position in fifty (or one) may be
    over the limit by up to half of it.  The largest |difference| that was held is recorded under `case`."""
    from tests.conftest import record_worst
    from tests.util import collect
    got = collect(steps, out_dir, vocab)
    worst, lim_of_worst, excused, total, slightly = 0.0, 0.0, 0, 0, 0
    for rid, rows in got.items():
        base = limits(dtype, want[rid])
        first_close = min(close.get(rid) or [1 << 30]) if (close is not None and dtype != "float32") else 1 << 30
        for pos, row in rows.items():
            total += 1
            lim = base if floor is None else max(base, 3.0 * float(floor[rid][pos]))
            w = want[rid][pos]
            diff = (torch.from_numpy(row.copy()) - w).abs().max().item()
            if diff > lim and pos >= first_close:
                excused += 1
                continue
            if dtype != "float32" and lim < diff <= 1.5 * lim:
                slightly += 1             # a rounding outlier: few are allowed, none beyond one and a half times the limit
                continue
            assert diff <= lim, f"{rid} position {pos}: |diff| {diff:.3e} > {lim:.3e}"
            if diff >= worst:
                worst, lim_of_worst = diff, lim
            if dtype == "float32" and floor is None:
                assert int(row.argmax()) == int(w.argmax())
    assert excused <= EXCUSED * total, f"{excused} of {total} positions differ"
    assert slightly <= max(1, 0.02 * total), f"{slightly} of {total} positions are over the limit"
    if case is not None:
        record_worst(case, dtype, worst, lim_of_worst)
    return got, worst


W64: dict = {}         # configuration tag -> the stored weights as float64 (set by the fixture)


def stored(weights: dict) -> dict:
    """The values that the folder holds (bfloat16), as float64: both sides compute from the same numbers."""
    return {k: v.to(torch.bfloat16).to(torch.float64) for k, v in weights.items()}


@pytest.fixture(scope="module", params=sorted(CONFIGS))
def setup(request, tmp_path_factory):
    tag = request.param
    c = CONFIGS[tag]
    weights = make_weights(c, seed=5)
    folder = write_folder(tmp_path_factory.mktemp(f"guronex_{tag}"), c, weights)
    w = W64[tag] = stored(weights)
    seqs = {f"r{i}": random_tokens(n, c["vocab"], seed=20 + i) for i, n in enumerate(LENGTHS[tag])}
    both = {rid: oracle(c, w, t) for rid, t in seqs.items()}
    want = {rid: v[0] for rid, v in both.items()}
    close = {rid: v[1] for rid, v in both.items()}
    assert all(v.abs().max() > 1.0 for v in want.values())     # logits of order one, not a flat model
    return tag, folder, seqs, (want, close)


def replay(folder, tag, dtype, steps, out_dir, max_tokens, **switches):
    from jax_vllm_b200.engine.replay import Replayer
    rep = Replayer(folder, dtype, out_dir, max_tokens=max_tokens, page_size=PAGE[tag], **switches)
    rep.run_stream(json.dumps(s) for s in steps)
    rep.cache.check()
    assert not rep.cache.live
    return rep


class Routes:
    """Records which experts the engine chose, call by call (a context manager around a replay), and puts them
    back together per request: {request: [one [tokens, top] tensor per routed layer]}."""

    def __enter__(self):
        from jax_vllm_b200 import ops
        self.ops, self.orig, self.calls = ops, ops.moe_route, []

        def recording(*a, **k):
            ids, weights = self.orig(*a, **k)
            self.calls.append(ids.cpu().long())
            return ids, weights
        ops.moe_route = recording
        return self

    def __exit__(self, *exc):
        self.ops.moe_route = self.orig
        return False

    def per_request(self, steps, n_routed):
        assert len(self.calls) == n_routed * len(steps)          # every step ran every routed layer once, eagerly
        out = {}
        for k, s in enumerate(steps):
            at = 0
            for e in s["entries"]:
                n = len(e["tokens"])
                for layer in range(n_routed):
                    out.setdefault(e["id"], [[] for _ in range(n_routed)])[layer].append(self.calls[k * n_routed + layer][at:at + n])
                at += n
        return {rid: [torch.cat(parts) for parts in layers] for rid, layers in out.items()}


def replay_bf16_following_the_engines_choice(folder, tag, c, w, seqs, steps, out_dir, max_tokens, case):
    """bfloat16, every position held: the plain implementation is made to take the experts that the engine took,
    and the engine may have taken others than the plain router only where the router logits nearly tie."""
    with Routes() as routes:
        rep = replay(folder, tag, "bfloat16", steps, out_dir, max_tokens)
    n_routed = sum(1 for ly in c["layers"] if ly["mlp"] is not None)
    taken = routes.per_request(steps, n_routed)
    want, floor = {}, {}
    to16 = lambda t: t.to(torch.bfloat16).to(t.dtype)
    for rid, forced in taken.items():
        margins, free = [], []
        toks = seqs[rid][:forced[0].shape[0]] if forced else seqs[rid]
        exact = gp.forward(c, w, toks, margins=margins, forced=forced, free=free)
        want[rid] = exact.to(torch.float32)
        # how far the rounding of the branches' inputs to 16 bits alone moves each position (same experts)
        floor[rid] = (gp.forward(c, w, toks, forced=forced, round_inputs=to16) - exact).abs().max(dim=1).values
        for layer in range(n_routed):
            differs = (forced[layer].sort(dim=1).values != free[layer].sort(dim=1).values).any(dim=1)
            assert (margins[layer][differs] < CLOSE_CALL).all(), f"{rid}: the engine chose other experts far from a tie"
    compare(steps, out_dir, c["vocab"], want, "bfloat16", case=case, floor=floor)
    return rep


# ------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("experts,top,groups,width", [(8, 3, (4, 2), 64), (40, 5, (5, 2), 80), (6, 1, (1, 1), 96),
                                                      (12, 3, (3, 3), 50), (16, 4, None, 128), (64, 6, (8, 3), 256)])
def test_router_alone(experts, top, groups, width):
    from jax_vllm_b200 import ops
    g = torch.Generator().manual_seed(experts + top)
    x = torch.randn((70, width), generator=g)
    w = torch.randn((experts, width), generator=g) * (2.0 / width ** 0.5)
    rt = {"experts": experts, "top": top}
    if groups is not None:
        rt["groups"] = {"count": groups[0], "keep": groups[1]}
    chosen, weight = gp.route(x.double(), w.double(), rt)
    n, keep = groups or (1, 1)
    ids, wts = ops.moe_route(ops.linear(x.cuda(), w.cuda(), torch.float32), top, n, keep, False)
    assert ids.cpu().tolist() == chosen.tolist()                # largest first, as the oracle's topk gives them
    assert torch.allclose(wts.cpu().double(), weight, rtol=1e-5, atol=1e-7)
    assert not torch.allclose(wts.sum(dim=1).cpu(), torch.ones(70))          # the scores are not renormalised
    if groups is not None and groups[1] < min(top, groups[0]):    # more groups could be hit than are kept
        free, _ = gp.route(x.double(), w.double(), {"experts": experts, "top": top})
        assert free.tolist() != chosen.tolist()                 # the groups do restrict the choice in this case


@pytest.mark.parametrize("W,E,ff,top,tensor_cores", [(72, 10, 24, 3, False), (256, 10, 136, 3, True)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_routed_experts_alone(dtype, W, E, ff, top, tensor_cores):
    """The part by itself: route, order by expert, two grouped products (on CUDA cores; in bfloat16 at sizes
    from 128 on the tcgen05 product, also with an expert size that is no multiple of its tiles), weighted sum by
    the reader."""
    from jax_vllm_b200.config.model_spec import RoutedExpertsSpec
    from jax_vllm_b200.parts import BuildContext
    from jax_vllm_b200.parts.routed_experts import RoutedExperts
    g = torch.Generator().manual_seed(3)
    tensors = {"b.f.router": torch.randn((E, W), generator=g) * 0.3}
    for e in range(E):
        tensors[f"b.f.e{e}.up"] = torch.randn((ff, W), generator=g) / W ** 0.5
        tensors[f"b.f.e{e}.down"] = torch.randn((W, ff), generator=g) / ff ** 0.5
    tensors = {k: v.to(torch.bfloat16) for k, v in tensors.items()}
    part = RoutedExperts(RoutedExpertsSpec(W, E, top, ff, n_groups=5, keep_groups=3, prefix="f"), "b",
                         BuildContext(dtype=dtype, device=torch.device("cuda")))
    assert set(part.tensor_specs()) == set(tensors)
    part.bind({k: v.cuda() for k, v in tensors.items()})
    assert part._tensor_cores() == (tensor_cores and dtype == torch.bfloat16)
    ml = {"router": {"experts": E, "top": top, "groups": {"count": 5, "keep": 3}}}
    w64 = {k: v.double() for k, v in tensors.items()}
    for n in (1, 5, 97, 700):                                   # fewer rows than experts, and several tiles an expert
        x = torch.randn((n, W), generator=g).to(torch.bfloat16)
        got = part.forward(x.cuda().to(dtype), None).tensor().cpu().double()
        want = gp.routed_experts(x.double(), w64, "b.f", ml)
        sure = gp.route_margin(x.double(), w64["b.f.router"], ml["router"]) > 1e-3
        lim = 1e-5 if dtype == torch.float32 else 3e-2
        assert sure.sum() > 0.9 * n
        assert (got - want)[sure].abs().max() <= lim * max(1.0, want.abs().max().item())
    from jax_vllm_b200 import ops
    ops.check_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_branch_norm_add_alone(dtype):
    from jax_vllm_b200 import ops
    g = torch.Generator().manual_seed(1)
    for hidden in (64, 100, 1000):
        h = torch.randn((9, hidden), generator=g)
        y = torch.randn((9, hidden), generator=g).to(dtype)
        w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16)
        want = h.double() + 0.4 * gp.rms_norm(y.double(), w.double(), 1e-5)
        hd = h.cuda()
        x = ops.branch_norm_add(hd, y.cuda(), w.cuda(), 1e-5, 0.4, x_dtype=dtype)
        assert (hd.cpu().double() - want).abs().max() < 2e-6
        assert torch.equal(x.cpu(), hd.cpu().to(dtype))          # the copy is the stream, rounded once
        # the same branch as weighted rows of a longer tensor
        rows = torch.randn((30, hidden), generator=g).to(dtype)
        pick = torch.randint(0, 30, (9, 3), generator=g, dtype=torch.int32)
        coef = torch.rand((9, 3), generator=g)
        branch = (coef.double()[:, :, None] * rows.double()[pick.long()]).sum(dim=1)
        want = h.double() + 0.4 * gp.rms_norm(branch, w.double(), 1e-5)
        hd = h.cuda()
        ops.branch_norm_add(hd, ops.PickedRows(rows.cuda(), pick.cuda(), coef.cuda()), w.cuda(), 1e-5, 0.4)
        assert (hd.cpu().double() - want).abs().max() < 2e-6
        assert (ops.PickedRows(rows.cuda(), pick.cuda(), coef.cuda()).tensor().cpu().double() - branch).abs().max() < 1e-5


def test_token_gate_alone():
    from jax_vllm_b200 import ops
    g = torch.Generator().manual_seed(2)
    z = torch.randn((11, 6), generator=g) * 3
    table = torch.randn((20, 30), generator=g)
    tokens = torch.randint(0, 20, (11,), generator=g, dtype=torch.int32)
    got = ops.token_gate(z.cuda(), tokens.cuda(), table.cuda(), 12).cpu().double()
    want = gp.gelu_tanh(z.double()) * table.double()[tokens.long()][:, 12:18]
    assert (got - want).abs().max() < 1e-6
    ops.token_gate(z.cuda(), torch.full((11,), 20, dtype=torch.int32).cuda(), table.cuda(), 0)
    with pytest.raises(ops.KernelError, match="token id outside"):
        ops.check_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_prepare_alone(dtype):
    """The cache row [normed latent | rotated key part] and the rotated query parts, at positions far from 0, on
    pages given in a scrambled order."""
    from jax_vllm_b200 import ops
    H, dp, dr, dc, P = 3, 8, 12, 20, 4
    dk = dc + dr
    g = torch.Generator().manual_seed(4)
    n = 7
    positions = torch.tensor([0, 1, 5, 1001, 1002, 1003, 30000], dtype=torch.int32)
    entry = torch.tensor([0, 0, 0, 1, 1, 1, 2], dtype=torch.int32)
    row = torch.randn((n, H * (dp + dr) + dk + 5), generator=g).to(dtype)
    norm_w = (1 + 0.1 * torch.randn(dc, generator=g)).to(torch.bfloat16)
    base = 1e4
    inv_freq = (base ** (-torch.arange(0, dr, 2, dtype=torch.float32) / dr))
    width = 30000 // P + 1
    table = torch.full((3, width), -1, dtype=torch.int32)
    table[0, 0], table[0, 1], table[1, 250], table[2, 7500] = 5, 2, 0, 3
    cache = torch.full((6, P, 1, dk), float("nan"), dtype=dtype)
    cache_d = cache.cuda()
    q = torch.zeros((n, H * dk), dtype=dtype).cuda()
    ops.latent_prepare(row.cuda(), 0, H * (dp + dr), None, q, positions.cuda(), entry.cuda(), table.cuda(),
                       inv_freq.cuda(), norm_w.cuda(), 1e-5, cache_d, H, dp, dr, dc)
    ops.check_status()
    r64 = row.double()
    kv = r64[:, H * (dp + dr):H * (dp + dr) + dk]
    c = gp.rms_norm(kv[:, :dc], norm_w.double(), 1e-5)
    kr = gp.rotate(kv[:, dc:], positions, base)
    tol = 3e-5 if dtype == torch.float32 else 2e-2       # float32 angles at position 30000 carry about 1e-3 / 2^-10
    where = [(5, 0), (5, 1), (2, 1), (0, 1), (0, 2), (0, 3), (3, 0)]
    got = cache_d.cpu().double()
    for t, (page, slot) in enumerate(where):
        assert (got[page, slot, 0, :dc] - c[t]).abs().max() < tol
        assert (got[page, slot, 0, dc:] - kr[t]).abs().max() < (tol if positions[t] < 2000 else 40 * tol)
    written = torch.zeros((6, P), dtype=torch.bool)
    for page, slot in where:
        written[page, slot] = True
    assert torch.isnan(got[~written]).all()                  # nothing else was touched
    qr = gp.rotate(r64[:, :H * (dp + dr)].reshape(n, H, dp + dr)[:, :, dp:].transpose(0, 1), positions, base).transpose(0, 1)
    gq = q.cpu().double().reshape(n, H, dk)
    assert (gq[:6, :, dc:] - qr[:6]).abs().max() < tol
    assert (gq[:, :, :dc] == 0).all()                        # the latent part belongs to the batched product


@pytest.mark.parametrize("heads,dk,dv", [(3, 48, 40), (5, 96, 72), (2, 384, 320), (16, 576, 512), (70, 24, 16), (1, 160, 128)])
def test_latent_tensor_core_attention_alone(heads, dk, dv):
    """csrc/attn_latent_mma.cu against the CUDA-core kernel (32-bit arithmetic) on the same bfloat16 rows: three
    entries with earlier context (a prompt portion over several tiles, a short one, a single token split along its
    keys), pages in a scrambled order, unowned places filled with NaN."""
    from jax_vllm_b200 import ops
    g = torch.Generator().manual_seed(heads * dk)
    P, n_pages = 8, 64
    ctx, new = [37, 0, 130], [45, 3, 1]
    cache = torch.full((n_pages, P, 1, dk), float("nan"), dtype=torch.bfloat16)
    width = max(-(-(c + q) // P) for c, q in zip(ctx, new))
    table = torch.full((3, width), -1, dtype=torch.int32)
    free = torch.randperm(n_pages, generator=g).tolist()
    for e, (c, q) in enumerate(zip(ctx, new)):
        for i in range(-(-(c + q) // P)):
            table[e, i] = free.pop()
            fill = min(P, c + q - i * P)
            cache[table[e, i], :fill] = torch.randn((fill, 1, dk), generator=g).to(torch.bfloat16)
    n = sum(new)
    q = (torch.randn((n, heads * dk), generator=g) * 0.5).to(torch.bfloat16).cuda()
    cu = torch.tensor([0, 45, 48, 49], dtype=torch.int32).cuda()
    start = torch.tensor(ctx, dtype=torch.int32).cuda()
    cache_d, table_d = cache.cuda(), table.cuda()
    tpt = ops.attn_latent_mma_tokens_per_tile(heads)
    work = torch.tensor([(e, t) for e in (0, 1) for t in range(0, new[e], tpt)], dtype=torch.int32).cuda()
    spt = ops.attn_simt_tokens_per_tile(heads, 1)
    work_s = torch.tensor([(e, t) for e in (0, 1) for t in range(0, new[e], spt)], dtype=torch.int32).cuda()
    dwork = torch.tensor([(2, 0)], dtype=torch.int32).cuda()
    scale = dk ** -0.5
    got = torch.zeros((n, heads * dv), dtype=torch.bfloat16).cuda()
    want = torch.zeros_like(got)
    assert ops.attn_latent_mma_supports(torch.bfloat16, dk, dv)
    ops.attn_latent_mma(q, q.stride(0), got, cache_d, table_d, cu, start, work, work.shape[0], heads, dk, dv, scale)
    ops.attn_latent_mma(q, q.stride(0), got, cache_d, table_d, cu, start, dwork, 1, heads, dk, dv, scale,
                        split_size=32, n_splits=5)
    ops.attn_simt(q, q.stride(0), want, cache_d, cache_d, table_d, cu, start, work_s, work_s.shape[0], heads, 1, dk, 0,
                  scale, v_dim=dv)
    ops.attn_simt(q, q.stride(0), want, cache_d, cache_d, table_d, cu, start, dwork, 1, heads, 1, dk, 0, scale,
                  split_size=32, n_splits=5, v_dim=dv)
    ops.check_status()
    assert torch.isfinite(got.float()).all()
    assert (got.float() - want.float()).abs().max() < 2e-2          # P is rounded to bfloat16 before it meets V


# --------------------------------------------------------------- models of several sizes
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_each_request_alone_and_whole(setup, dtype, tmp_path):
    tag, folder, seqs, want = setup
    for rid, toks in seqs.items():
        steps = whole(rid, toks)
        if dtype == "bfloat16":
            replay_bf16_following_the_engines_choice(folder, tag, CONFIGS[tag], W64[tag], seqs, steps, tmp_path / rid, 128 * 3,
                                                     f"guronex {tag}, whole")
            continue
        replay(folder, tag, dtype, steps, tmp_path / rid, max_tokens=128 * 3)
        compare(steps, tmp_path / rid, CONFIGS[tag]["vocab"], want[0], dtype, case=f"guronex {tag}, whole", close=want[1])


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_last_tokens_one_by_one(setup, dtype, graphs, tmp_path):
    """Prefill against token-by-token decoding, eagerly and from the captured graph."""
    tag, folder, seqs, want = setup
    steps = prefix_then_single("r0", seqs["r0"], tail=24)
    if dtype == "bfloat16" and not graphs:
        replay_bf16_following_the_engines_choice(folder, tag, CONFIGS[tag], W64[tag], seqs, steps, tmp_path, 256,
                                                 f"guronex {tag}, decoding")
        return
    rep = replay(folder, tag, dtype, steps, tmp_path, max_tokens=256, cuda_graphs=graphs)
    assert any(m["replayed_graph"] for m in rep.records) == graphs
    compare(steps, tmp_path, CONFIGS[tag]["vocab"], want[0], dtype, case=f"guronex {tag}, decoding", close=want[1])


@pytest.mark.parametrize("sizes", [(2,), (7, 2, 13, 1, 1, 5), (33, 3, 64)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_of_changing_size(setup, dtype, sizes, tmp_path):
    tag, folder, seqs, want = setup
    steps = portions("r2", seqs["r2"], sizes)
    if dtype == "bfloat16":
        replay_bf16_following_the_engines_choice(folder, tag, CONFIGS[tag], W64[tag], seqs, steps, tmp_path, 256,
                                                 f"guronex {tag}, portions {sizes}")
        return
    replay(folder, tag, dtype, steps, tmp_path, max_tokens=256)
    compare(steps, tmp_path, CONFIGS[tag]["vocab"], want[0], dtype, case=f"guronex {tag}, portions {sizes}", close=want[1])


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
    if dtype == "bfloat16":
        rep = replay_bf16_following_the_engines_choice(folder, tag, CONFIGS[tag], W64[tag], seqs, steps, tmp_path, live3,
                                                       f"guronex {tag}, side by side")
    else:
        rep = replay(folder, tag, dtype, steps, tmp_path, max_tokens=live3)
        compare(steps, tmp_path, CONFIGS[tag]["vocab"], want[0], dtype, case=f"guronex {tag}, side by side", close=want[1])
    assert sum(m["pages_allocated"] for m in rep.records) > rep.cache.num_pages * len(rep.cache.groups)   # pages came back and went out again


def test_schedules_agree_with_each_other_in_32_bit(setup, tmp_path):
    """A position's logits do not depend on the cut, the batch or the pages beyond rounding."""
    from tests.util import collect
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
        assert abs(ga[pos] - gb[pos]).max() < 2e-5 and abs(ga[pos] - gc[pos]).max() < 2e-5


def test_trace_run_program(tmp_path):
    """bin/trace_run as a program on a Guronex folder: stdin steps, `done <step>` lines, files on disk, exit 0."""
    c = CONFIGS["ga"]
    weights = make_weights(c, seed=9)
    folder = write_folder(tmp_path / "model", c, weights)
    seqs = {f"r{i}": random_tokens(n, c["vocab"], seed=40 + i) for i, n in enumerate([40, 21, 33, 12])}
    want = {rid: gp.forward(c, stored(weights), t).to(torch.float32) for rid, t in seqs.items()}
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("far", [0, 1, 15, 16, 17, 255, 256])
def test_one_far_key_among_hundreds(far, dtype, tmp_path):
    """One layer without a feed-forward.  Token 1 stands at position `far` only (the first tokens, a page's last
    and first places); its key part is made large along the direction that the last token's query has, so that
    this one score stands out among 600.  The plain implementation's result changes greatly when the far token is
    taken away; the engine's must equal the result with it, whole, in portions and decoded."""
    c = config(50, 64, [layer(mixer(2, 16, 8, 16, 24, scale=1.0), None)], mult=1.0)
    w = make_weights(c, seed=11)
    w["embed"][1] = 6.0 * w["embed"][1] / w["embed"][1].norm() * 8
    w["embed"][2] = 6.0 * w["embed"][2] / w["embed"][2].norm() * 8
    # token 2 (the last one) asks for token 1: its plain query, through W_uk, points along token 1's latent
    w64 = stored(w)
    tokens = [3 + (i * 7) % 40 for i in range(600)]
    tokens[far], tokens[-1] = 1, 2
    c1, _ = gp.latent_and_rotated_key(w64["embed"][[1]], w64, "l0.mix", c["layers"][0]["mixer"], c["norm"]["eps"], torch.tensor([far]))
    uk = w64["l0.mix.uk"].reshape(2, 16, 24)
    target = torch.einsum("hdr,r->hd", uk, c1[0])                      # the plain key of token 1, per head
    x2 = w64["embed"][2]
    q = torch.zeros((2, 24, 64), dtype=torch.float64)
    q[:, :16, :] = 1.5 * target[:, :, None] * x2[None, None, :] / (x2 @ x2)
    w["l0.mix.q"] = q.reshape(48, 64).to(torch.float32)
    w64 = stored(w)
    with_key = gp.forward(c, w64, tokens).to(torch.float32)          # no routed layer: nothing hangs on a close call
    without = list(tokens)
    without[far] = 4
    gone = gp.forward(c, w64, without).to(torch.float32)
    assert (with_key[-1] - gone[-1]).abs().max() > 0.5                   # the far key decides the last logits
    want = {"r": with_key}
    for sizes, tail in ((None, 0), ((100, 3, 2), 0), (None, 9)):
        steps, out = special(tmp_path, c, w, tokens, dtype, sizes=sizes, tail=tail)
        compare(steps, out, 50, want, dtype, case=f"guronex one far key at {far}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_values_that_happen_to_be_one_or_equal(dtype, tmp_path):
    """One head, one expert of which one is chosen, a residual multiplier of 1, a token input of one column, rot_dim
    2, and plain, rotated and value sizes all different; then a multiplier far from 1 with equal sizes."""
    for k, c in enumerate((config(64, 48, [layer(mixer(1, 10, 2, 6, 14), moe(1, 1, 8)),
                                           layer(mixer(1, 10, 2, 6, 14, kv_from=0), moe(2, 2, 8, (2, 2)))], mult=1.0, side=1),
                           config(64, 32, [layer(mixer(2, 16, 16, 16, 16), moe(4, 2, 32, (2, 1)))], mult=0.05, side=16))):
        w = make_weights(c, seed=13 + k)
        tokens = random_tokens(45, 64, seed=14)
        logits, close = oracle(c, stored(w), tokens)
        # a token input of ONE column is normed to +-1 times its projection unless the column is tiny: there the
        # 32-bit rounding of the gate shows.  What the plain implementation itself loses in 32-bit is the floor.
        w32 = {name: v.to(torch.bfloat16).to(torch.float32) for name, v in w.items()}
        floor = (gp.forward(c, w32, tokens).double() - gp.forward(c, stored(w), tokens)).abs().max(dim=1).values
        for sizes in (None, (2,)):
            steps, out = special(tmp_path / str(k), c, w, tokens, dtype, sizes=sizes, page=8)
            compare(steps, out, 64, {"r": logits}, dtype, case=f"guronex sizes of one ({k})", close={"r": close},
                    floor={"r": floor} if dtype == "float32" else None)


# ----------------------------------------------------------- generation, scheduler, entry point
def plain_greedy(c, w, prompt, n):
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(gp.forward(c, w, seq)[-1].argmax()))
    return seq[len(prompt):]


def test_greedy_generation_through_the_entry_point(tmp_path):
    """make_driver + generate: the scheduler's portions, decode steps from captured graphs, sampling."""
    from jax_vllm_b200 import SamplingParams, generate, load_from_path, make_driver
    c = CONFIGS["ga"]
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
    c = CONFIGS["gb"]
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
