"""Pivinex on the GPU: every new mechanism alone against the plain implementation's function for it, then the
engine through the replay loop and through ``Engine.generate`` against the plain implementation of the whole
model, in 32-bit and in bfloat16, for four small configurations that differ in every size and option."""

import json
import math

import numpy as np
import pytest
import torch

import helpers as H
import pivinex_helpers as PH
from plain import pivinex_plain as PP

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
BOTH = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    from pyre_b200.kernels import ops as o
    return o


def close(got, want, dtype, what="", atol32=3e-6, rel16=1.6e-2):
    tol = dict(rtol=3e-5, atol=atol32) if dtype == torch.float32 else dict(rtol=rel16, atol=rel16)
    torch.testing.assert_close(got.double().cpu(), want.double().cpu(), msg=lambda m: f"{what}: {m}", **tol)


def bf16_exact(*shape, scale=1.0, seed=0):
    """Random fp64 values that bfloat16 holds exactly."""
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).double()


# --------------------------------------------------------------------------- the small kernels, each alone
@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("T,Hn,two", [(1, 96, True), (5, 92, False), (37, 1024, True), (3, 4100, True)])
def test_layer_norm_adds_the_branches_with_their_gains(ops, dtype, T, Hn, two):
    x = bf16_exact(T, Hn, seed=1) + 0.3
    a, f = bf16_exact(T, Hn, seed=2), bf16_exact(3, T, Hn, seed=3)      # a branch tensor, and a split product's parts
    g1, g2, w = (bf16_exact(Hn, seed=s).float() for s in (4, 5, 6))
    want_x = x + g1.double() * a + (g2.double() * f.sum(0) if two else 0)
    want_h = PP.layer_norm(want_x, w.double(), 1e-5)
    xd = x.float().cuda()
    terms = [(a.to(dtype).cuda(), g1.cuda())] + ([(ops.PartialSums(f.float().cuda(), dtype), g2.cuda())] if two else [])
    h = ops.add_layernorm(xd, ops.ScaledSum(terms, dtype), w.cuda(), 1e-5, dtype)
    close(xd, want_x, torch.float32, "stream", atol32=2e-5)
    close(h, want_h, dtype, "activations", atol32=2e-5)
    # gathered rows leave the stream alone; the stream itself normalised stays fp32
    rows = torch.tensor([T - 1, 0], dtype=torch.int32, device="cuda")
    before = xd.clone()
    close(ops.add_layernorm(xd, None, w.cuda(), 1e-5, dtype, rows=rows), want_h[[T - 1, 0]], dtype, "rows", atol32=2e-5)
    assert torch.equal(xd, before)
    s = ops.add_layernorm(xd, None, w.cuda(), 1e-5, torch.float32, act_dtype=dtype)
    assert s.dtype == torch.float32
    close(s, want_h, torch.float32, "stream norm", atol32=2e-5)
    close(ops.materialize(ops.ScaledSum(terms, dtype)), want_x - x, dtype, "materialized")


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("kind", ["silu", "gelu_tanh"])
def test_gated_activation(ops, dtype, kind):
    gu = bf16_exact(7, 2 * 50, scale=2.0, seed=9)
    g, u = gu[:, :50], gu[:, 50:]
    want = (PP.silu(g) if kind == "silu" else PP.gelu_tanh(g)) * u
    close(ops.act_mul(gu.to(dtype).cuda(), kind), want, dtype, kind)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("q_rank,rank,rope,rot,page,parts", [(40, 24, 8, 8, 16, 0), (20, 36, 12, 8, 8, 2), (96, 192, 32, 32, 32, 0),
                                                              (8, 16, 0, 0, 4, 3)])
def test_latent_norms_rotation_and_paged_write(ops, dtype, q_rank, rank, rope, rot, page, parts):
    T, n_pages = 9, 6
    W = q_rank + rank + rope
    row = -(-(rank + rope) // 16) * 16
    proj = bf16_exact(max(parts, 1), T, W, seed=11)
    full = proj.sum(0)
    wq, wc = bf16_exact(q_rank, seed=12) + 1, bf16_exact(rank, seed=13) + 1
    pos = torch.tensor([0, 1, 2, 3, 77, 78, 500, 511, 600])      # angles are fp32 in the engine: 600 x 2^-24 of error
    slots = torch.randperm(page * n_pages, generator=torch.Generator().manual_seed(rank))[:T]
    inv = (1000.0 ** (-torch.arange(0, rot, 2, dtype=torch.float64) / rot)).float() if rot else None
    cos = sin = None
    if rot:
        cos, sin = ops.rope_table(pos.int().cuda(), inv.cuda())
    cache = torch.full((n_pages, 1, 1, page, row), 7.0, dtype=dtype, device="cuda")
    src = ops.PartialSums(proj.float().cuda(), dtype) if parts else full.to(dtype).cuda()
    cq = ops.latent_prepare(src, 0, q_rank, q_rank, rank, rope, rot, wq.float().cuda(), wc.float().cuda(), 1e-5, cos, sin,
                            cache, slots.int().cuda(), page, dtype)
    close(cq, PP.rms_norm(full[:, :q_rank], wq, 1e-5), dtype, "query latent")
    want = torch.cat([PP.rms_norm(full[:, q_rank:q_rank + rank], wc, 1e-5),
                      PP.rotate_pairs(full[:, q_rank + rank:], pos, 1000.0, rot) if rope else full[:, :0]], dim=1)
    flat = cache.view(-1, row)
    close(flat[slots.cuda(), :rank + rope], want, dtype, "cache rows", atol32=2e-4)
    assert (flat[slots.cuda(), rank + rope:] == 0).all(), "the padding of a row is zero"
    untouched = torch.ones(page * n_pages, dtype=torch.bool)
    untouched[slots] = False
    assert (flat[untouched.cuda()] == 7.0).all(), "a row of no token was written"
    # the queries' rotated part
    nh, dq = 3, 10
    q = bf16_exact(T, nh * (dq + rope), seed=14)
    qa = torch.full((T, nh, row), 5.0, dtype=dtype, device="cuda")
    ops.latent_rotate_q(q.to(dtype).cuda(), qa, cos, sin, nh, dq, rope, rot, rank)
    if rope:
        close(qa[..., rank:rank + rope], PP.rotate_pairs(q.view(T, nh, dq + rope)[..., dq:], pos, 1000.0, rot), dtype, "rotated queries", atol32=2e-4)
    assert (qa[..., :rank] == 5.0).all() and (qa[..., rank + rope:] == 0).all()


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("mma", [False, True])
@pytest.mark.parametrize("T,Hn,K,N,xs,os_", [(5, 3, 16, 24, 24, 32), (130, 4, 32, 48, 48, 64), (70, 5, 20, 36, 32, 36), (1, 8, 64, 192, 96, 224),
                                             (300, 3, 72, 200, 80, 208)])
def test_a_product_per_head(ops, dtype, mma, T, Hn, K, N, xs, os_, monkeypatch):
    monkeypatch.setattr(ops, "USE_GROUPED_MMA", mma)
    x, w = bf16_exact(T, Hn, xs, seed=21), bf16_exact(Hn, N, K, seed=22)
    want = torch.einsum("thk,hnk->thn", x[..., :K], w)
    out = torch.full((T, Hn, os_), 3.0, dtype=dtype, device="cuda")
    ops.headwise_linear(x.to(dtype).cuda(), w.to(dtype).cuda(), out=out)
    close(out[..., :N], want, dtype, "into wider rows", atol32=2e-5, rel16=4e-2)
    assert (out[..., N:] == 3.0).all()
    close(ops.headwise_linear(x.to(dtype).cuda(), w.to(dtype).cuda()), want, dtype, "fresh", atol32=2e-5, rel16=4e-2)


def plain_latent_attention(qa, rows_of, positions, seqs, rank, kd, scale, window):
    """Per token: softmax over the visible cached rows of its sequence of (qa . row[:kd]) * scale, times row[:rank]."""
    T, nh, _ = qa.shape
    out = torch.zeros(T, nh, rank, dtype=torch.float64)
    for t in range(T):
        p = int(positions[t])
        lo = max(0, p - window + 1) if window else 0
        rows = rows_of[int(seqs[t])][lo:p + 1]
        s = qa[t, :, :kd] @ rows[:, :kd].T * scale
        out[t] = torch.softmax(s, dim=-1) @ rows[:, :rank]
    return out


def paged(rows_of, page, row, dtype, first_live=None, seed=0):
    """Sequences' rows on scattered pages of a pool; pages before ``first_live[b]`` are not there (-1) and the
    pool's other rows are NaN."""
    n_pages = sum(-(-r.shape[0] // page) for r in rows_of) + 3
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    pool = torch.full((n_pages, 1, 1, page, row), float("nan"), dtype=torch.float64)
    width = max(-(-r.shape[0] // page) for r in rows_of)
    table = torch.full((len(rows_of), width), -1, dtype=torch.int32)
    for b, r in enumerate(rows_of):
        for lp in range(-(-r.shape[0] // page)):
            if first_live is not None and lp < first_live[b]:
                continue
            pg = perm.pop()
            table[b, lp] = pg
            piece = r[lp * page:(lp + 1) * page]
            pool[pg, 0, 0, :piece.shape[0], :r.shape[1]] = piece
            pool[pg, 0, 0, :piece.shape[0], r.shape[1]:] = 0
    return pool.to(dtype).cuda(), table.cuda()


@pytest.mark.parametrize("kernel", ["exact32", "exact16", "mma"])
@pytest.mark.parametrize("nh,rank,rope,page,window", [(3, 24, 8, 16, 11), (7, 112, 16, 16, 33), (8, 192, 32, 32, 64), (72, 64, 16, 8, 0),
                                                      (5, 36, 12, 8, 7), (2, 272, 16, 16, 300), (4, 38, 12, 16, 9)])
def test_latent_attention_kernels(ops, kernel, nh, rank, rope, page, window):
    """Entries of many lengths in one launch (single tokens, portions that start in the middle of a page and of a
    window, one from position 0), each token against the plain softmax over exactly its window.  In every sequence
    one key just inside and one just outside the last token's window, one at a page's border and one far back stand
    out (their rows point along that token's query): a window, page or tile that is one off moves the output by its
    whole size.  Pages that a window has passed are absent."""
    dtype = torch.float32 if kernel == "exact32" else torch.bfloat16
    kd = rank + rope
    row = -(-kd // 16) * 16
    if kernel == "mma" and not ops.latent_mma_ok(dtype, row):
        pytest.skip("rows too wide for the tensor-core kernel")
    lens = [1, 1, 37, 2, 90, 130, 64, 5]              # new tokens per entry
    starts = [0, 250, 0, 97, 40, 3, 64, 1000]         # tokens cached before them
    g = torch.Generator().manual_seed(nh * 1000 + rank)
    rows_of, qa, positions, seqs = [], [], [], []
    scale = 1.0 / math.sqrt(kd)
    for b, (n, s0) in enumerate(zip(lens, starts)):
        total = s0 + n
        rows = (torch.randn(total, kd, generator=g) * 0.5).to(torch.bfloat16).double()
        q = (torch.randn(n, nh, kd, generator=g)).to(torch.bfloat16).double()
        last = total - 1
        lo = max(0, last - window + 1) if window else 0
        marks = [lo, lo - 1, (last // page) * page, (last // page) * page - 1, max(0, last - 200), 0]
        for k, j in enumerate(marks):
            if 0 <= j <= last:
                rows[j] = (q[-1, k % nh] * (1.5 + 0.2 * k)).to(torch.bfloat16).double()
        rows_of.append(rows)
        qa.append(q)
        positions += list(range(s0, total))
        seqs += [b] * n
    qa = torch.cat(qa)
    want = plain_latent_attention(qa, rows_of, positions, seqs, rank, kd, scale, window)
    first_live = [max(0, s0 - window + 1) // page if window else 0 for s0 in starts]
    pool, table = paged(rows_of, page, row, dtype, first_live, seed=rank)
    qa_d = torch.zeros(qa.shape[0], nh, row, dtype=dtype, device="cuda")
    qa_d[..., :kd] = qa.to(dtype).cuda()
    pos_d = torch.tensor(positions, dtype=torch.int32, device="cuda")
    seq_d = torch.tensor(seqs, dtype=torch.int32, device="cuda")
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32, device="cuda")
    if kernel != "mma":
        got = ops.latent_attention_exact(qa_d, pool[:, :, :, :, :], table, seq_d, pos_d, rank, rope, scale, window or None)
        close(got, want, dtype, kernel, atol32=2e-5, rel16=2e-2)
    else:
        tq = 64 // min(nh, 64)
        n_tiles = sum(-(-n // tq) for n in lens)
        for splits in (1, 3):
            got = ops.latent_attention_mma(qa_d, pool, table, cu, pos_d, n_tiles, rank, scale, window or None, n_splits=splits)
            assert torch.isfinite(got).all(), f"{splits} shares: non-finite outputs"
            close(got, want, dtype, f"mma, {splits} shares", rel16=2.5e-2)
        # entries of more than two tokens left to another kernel: their rows stay as they were
        out = torch.full((qa.shape[0], nh, rank), 9.0, dtype=dtype, device="cuda")
        short = sum(-(-n // tq) for n in lens if n <= 2)
        ops.latent_attention_mma(qa_d, pool, table, cu, pos_d, short, rank, scale, window or None, max_len=2, out=out)
        at = 0
        for n in lens:
            if n <= 2:
                close(out[at:at + n], want[at:at + n], dtype, "short entries only", rel16=2.5e-2)
            else:
                assert (out[at:at + n] == 9.0).all()
            at += n
    ops.check_device_errors()


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("mma", [False, True])
@pytest.mark.parametrize("T,Hn,ff,E,ident,top,scale", [(1, 96, 64, 5, 1, 2, 1.0), (77, 92, 24, 3, 2, 3, 0.7), (300, 256, 128, 8, 0, 2, 1.5),
                                                       (9, 64, 32, 4, 0, 1, 2.5), (40, 128, 16, 1, 3, 2, 1.0), (700, 128, 192, 4, 1, 2, 1.0)])
def test_routed_feed_forward_step_by_step(ops, dtype, mma, T, Hn, ff, E, ident, top, scale, monkeypatch):
    """Router (scores over all outputs, a correction that only the choice sees, weights not renormalised), the sort by
    expert, both products per expert and the weighted sum, outputs without weights included, against the plain
    functions; the inputs are drawn again until no choice is a close call."""
    monkeypatch.setattr(ops, "USE_GROUPED_MMA", mma)
    n_out = E + ident
    router = {"experts": E, "identity": ident, "top": top, "scale": scale}
    for seed in range(50):
        w = {"p.router": bf16_exact(n_out, Hn, scale=0.3, seed=seed), "p.correction": bf16_exact(n_out, scale=0.05, seed=seed + 100)}
        h = bf16_exact(T, Hn, seed=seed + 200)
        margins = []
        pick, weight = PP.route(h, w, "p.", router, margins)
        if not margins or min(margins) > 2e-3:
            break
    for e in range(E):
        w[f"p.e{e}.gate"], w[f"p.e{e}.up"], w[f"p.e{e}.down"] = (bf16_exact(ff, Hn, scale=0.08, seed=7 * e + 1), bf16_exact(ff, Hn, scale=0.08, seed=7 * e + 2),
                                                                bf16_exact(Hn, ff, scale=0.08, seed=7 * e + 3))
    hd = h.to(dtype).cuda()
    idx, wt = ops.route(hd, w["p.router"].float().cuda(), w["p.correction"].float().cuda(), top, scale)
    assert torch.equal(idx.cpu().long().sort(-1).values, pick.sort(-1).values), "the chosen outputs"
    order = idx.cpu().long().argsort(-1)
    close(wt.cpu().gather(-1, order), weight.gather(-1, pick.argsort(-1)), torch.float32, "weights", atol32=1e-6)
    offsets, place_of, src = ops.group_pairs(idx, E)
    off, po, sr = offsets.cpu().tolist(), place_of.cpu().view(-1).tolist(), src.cpu().tolist()
    flat = idx.cpu().view(-1).tolist()
    assert off[0] == 0 and off[-1] == sum(1 for e in flat if e < E)
    seen = set()
    for p, e in enumerate(flat):
        if e >= E:
            assert po[p] == -1
        else:
            assert off[e] <= po[p] < off[e + 1] and po[p] not in seen and sr[po[p]] == p // top
            seen.add(po[p])
    part = PartFor(ops, dtype, Hn, ff, E, ident, top, scale, w)
    got = part.forward(None, hd)
    got = got.parts.sum(0) if isinstance(got, ops.PartialSums) else got
    want = PP.moe_ffn(h, w, "p.", {"router": router})
    close(got, want, dtype, "routed feed-forward", atol32=2e-5, rel16=3e-2)


def PartFor(ops, dtype, Hn, ff, E, ident, top, scale, w):
    from pyre_b200.parts.base import PartSpec, load_part, make_part
    part = make_part("ffn", PartSpec("routed_mlp", {"width": Hn, "intermediate": ff, "n_experts": E, "n_identity": ident, "top": top,
                                                    "scale": scale}), dtype, "cuda")
    tensors = {}
    for name, spec in part.tensors().items():
        t = w["p." + name]
        tensors[name] = t.to(torch.float32 if spec.role == "vector" else dtype).cuda()
    load_part(part, tensors)
    return part


# --------------------------------------------------------------------------- the engine against the plain model
LENGTHS = {"A": [1, 2, 17, 33, 70, 130], "B": [5, 31, 97, 150], "C": [3, 63, 64, 65, 200], "D": [2, 47, 129]}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for n, (name, raw) in enumerate(PH.PIV.items()):
        d = tmp_path_factory.mktemp(f"pivinex_{name}")
        PH.make_pivinex_dir(d, raw, seed=500 + n)
        reqs = {f"{name}{i}": PH.decided_ids(d, L, seed=13 * n + i) for i, L in enumerate(LENGTHS[name])}
        plain = {rid: PH.plain_logits(d, ids) for rid, ids in reqs.items()}
        sq, cnt = 0.0, 0
        for rid, ids in reqs.items():
            e = PH.plain_logits(d, ids, lowp=True) - plain[rid]
            sq, cnt = sq + float((e ** 2).sum()), cnt + e.size
        out[name] = (d, reqs, plain, math.sqrt(sq / cnt))
    return out


def run(models, name, dtype, steps, what, want=None):
    d, reqs, plain, lowp_rms = models[name]
    got = H.run_trace_in_process(d, dtype, steps, H.max_live_tokens(steps), PH.PIV_PAGE_SIZE[name])
    PH.compare(got, want or plain, dtype, what, lowp_rms)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_prompts(models, name, dtype):
    run(models, name, dtype, H.trace_whole(models[name][1]), "whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_prefill_then_token_by_token(models, name, dtype):
    steps = []
    for k, (rid, ids) in enumerate(models[name][1].items()):
        # most of it in one step and the rest one by one (a window passes over decoded tokens); every third request
        # one by one from its first token
        steps += H.trace_decode_tail(rid, ids, len(ids) if k % 3 == 2 else 32, first_step=len(steps))
    run(models, name, dtype, steps, "decode")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_portions_down_to_two_tokens(models, name, dtype):
    steps = []
    for k, (rid, ids) in enumerate(models[name][1].items()):
        sizes = [[2, 9, 3, 17, 2, 31], [5, 2, 16, 8, 64], [24, 2, 2, 7, 1, 70]][k % 3]
        steps += H.trace_portions(rid, ids, sizes, first_step=len(steps))
    run(models, name, dtype, steps, "portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_mixed_batches_reuse_pages(models, name, dtype):
    """Every request twice under other names, at most four alive: later ones get the pages (filled with NaN when
    they were given back, by a window or at the end) that earlier ones held, and must come out as each alone."""
    d, reqs, plain, _ = models[name]
    many = {f"{rid}r{rep}": ids for rep in range(2) for rid, ids in reqs.items()}
    steps = H.trace_mixed(many, seed=21, max_live=4, portion=(2, 40))
    run(models, name, dtype, steps, "mixed", {f"{rid}r{rep}": plain[rid] for rep in range(2) for rid in reqs})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_long_decoding(models, name, dtype):
    """220 tokens, the last 150 or more one by one (captured decode steps), two requests side by side: every window
    passes over decoded tokens several times and gives pages back on the way."""
    d, _reqs, _plain, lowp_rms = models[name]
    reqs = {f"long{i}": PH.decided_ids(d, n, seed=90 + i) for i, n in enumerate([220, 190])}
    steps = [{"step": 0, "entries": [{"id": r, "tokens": ids[:70 - 30 * i], "want": [0]} for i, (r, ids) in enumerate(reqs.items())], "end": []}]
    at = {r: 70 - 30 * i for i, r in enumerate(reqs)}
    while any(at[r] < len(reqs[r]) for r in reqs):
        entries = [{"id": r, "tokens": [reqs[r][at[r]]], "want": [0]} for r in reqs if at[r] < len(reqs[r])]
        for e in entries:
            at[e["id"]] += 1
        steps.append({"step": len(steps), "entries": entries, "end": [e["id"] for e in entries if at[e["id"]] == len(reqs[e["id"]])]})
    got = H.run_trace_in_process(d, dtype, steps, H.max_live_tokens(steps), PH.PIV_PAGE_SIZE[name])
    want = {}
    for i, (r, ids) in enumerate(reqs.items()):
        full = PH.plain_logits(d, ids)
        want[r] = np.concatenate([full[:1], full[70 - 30 * i:]])
    PH.compare(got, want, dtype, "long decoding", lowp_rms)


@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_engine(models, name):
    """``Engine.generate`` (scheduler, portions of prompts, captured decode steps, sampler) gives the tokens that
    the plain implementation's argmax gives, in 32-bit; a cache too small for all requests at once makes the
    scheduler preempt and recompute."""
    from pyre_b200.engine.engine import Engine
    from pyre_b200.sampling import SamplingParams
    d, _reqs, _plain, _ = models[name]
    raw = PH.PIV[name]
    prompts = [H.random_ids(raw["vocab"], n, seed=40 + n) for n in (15, 16, 3, 30)]
    new = 12
    engine = Engine(str(d), dtype="float32", page_size=16, num_pages=5, max_num_seqs=3, max_num_batched_tokens=32, prefill_chunk=20)
    outs = engine.generate(prompts, SamplingParams(max_new_tokens=new, return_logits=True))
    for p, o in zip(prompts, outs):
        ids = list(p)
        for k in range(new):
            logits = PH.plain_logits(d, ids)[-1]
            top2 = np.sort(logits)[-2:]
            np.testing.assert_allclose(o.logits[k], logits, rtol=2e-4, atol=3e-5)
            if top2[1] - top2[0] > 1e-4:
                assert o.token_ids[k] == int(logits.argmax()), f"token {k} of a prompt of {len(p)}"
            ids.append(o.token_ids[k])
    assert json.dumps(engine.stats())
