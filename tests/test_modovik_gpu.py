"""Modovik on the GPU: every new mechanism alone against the plain implementation's function for it, then the
engine through the replay loop and through ``Engine.generate`` against the plain implementation of the whole
model, in 32-bit and in bfloat16, for four small configurations that differ in every size and option."""

import json
import math

import numpy as np
import pytest
import torch

import helpers as H
import modovik_helpers as MH
from plain import modovik_plain as MP

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def ops():
    from pyre_b200.kernels import ops as o
    return o


def close(got, want, dtype, what="", atol32=3e-6):
    tol = dict(rtol=3e-5, atol=atol32) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=1.6e-2)
    torch.testing.assert_close(got.double().cpu(), want.double().cpu(), msg=lambda m: f"{what}: {m}", **tol)


# --------------------------------------------------------------------------- the small kernels, each alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,Hn", [(1, 96), (5, 92), (37, 1024), (3, 4100)])
def test_norm_on_a_branch_output_is_added_to_the_stream(ops, dtype, T, Hn):
    g = torch.Generator(device="cuda").manual_seed(T * Hn)
    x = torch.randn(T, Hn, device="cuda", generator=g)
    y = (torch.randn(T, Hn, device="cuda", generator=g) * 3).to(dtype)
    w = 1.0 + 0.1 * torch.randn(Hn, device="cuda", generator=g)
    want = x.double() + MP.rms_norm(y.double(), w.double(), 1e-5)
    x1 = x.clone()
    nxt = ops.norm_add(x1, y, w, 1e-5, dtype, want_next=True)
    close(x1, want, torch.float32, "stream")
    if dtype == torch.float32:
        assert nxt is x1
    else:
        assert torch.equal(nxt, x1.to(dtype))
    # the same from fp32 partial sums of a split product
    parts = torch.randn(3, T, Hn, device="cuda", generator=g)
    x2 = x.clone()
    assert ops.norm_add(x2, ops.PartialSums(parts.contiguous(), dtype), w, 1e-5, dtype) is None
    close(x2, x.double() + MP.rms_norm(parts.double().sum(0), w.double(), 1e-5), torch.float32, "partials")
    assert ops.cast_rows(x, dtype).dtype == dtype and torch.equal(ops.cast_rows(x, dtype), x.to(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_activations(ops, dtype):
    z = (torch.linspace(-12, 12, 4099, device="cuda") * 1.0).to(dtype).reshape(1, -1)
    close(ops.activation(z, "gelu_tanh"), MP.gelu_tanh(z.double()), dtype, "gelu")
    close(ops.activation(z, "silu"), MP.silu(z.double()), dtype, "silu")
    with pytest.raises(ops.UnsupportedSize):
        ops.activation(z, "relu")


@pytest.mark.parametrize("M,N,K", [(300, 512, 256), (2048, 1000, 320), (129, 2048, 64), (640, 264, 1024), (8, 512, 256), (200, 96, 92)])
def test_product_with_gelu_in_its_epilogue(ops, M, N, K):
    """act(x W^T) of a prompt portion with the activation in the product's epilogue gives what the product followed
    by the activation kernel gives (the activation reads the product rounded to bfloat16 either way); few tokens,
    split products and sizes the tensor-core product does not take run the two kernels."""
    g = torch.Generator(device="cuda").manual_seed(M + N)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda", generator=g) * K ** -0.5 * 2).to(torch.bfloat16)
    got = ops.linear_act(x, w, "gelu_tanh")
    two = ops.activation(ops.materialize(ops.linear(x, w)), "gelu_tanh")
    want = MP.gelu_tanh((x.double() @ w.double().t()).to(torch.bfloat16).double())
    assert got.shape == (M, N) and got.dtype == torch.bfloat16
    close(got, want, torch.bfloat16, "fused")
    close(two, want, torch.bfloat16, "two kernels")
    assert (got.float() - two.float()).abs().max() <= 2 ** -6 * two.float().abs().max()
    ops.check_device_errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,dk,dv,rot,page,write", [(4, 2, 32, 16, 8, 16, True), (5, 5, 24, 40, 0, 8, True),
                                                         (3, 1, 64, 64, 64, 4, True), (6, 2, 80, 112, 32, 16, True),
                                                         (2, 1, 144, 64, 16, 16, True), (6, 3, 48, 20, 48, 16, False)])
def test_head_norm_rotation_and_paged_write(ops, dtype, nh, nkv, dk, dv, rot, page, write):
    """Queries and keys normed per head, their leading dims rotated, keys and values written to rows of one size
    (zero beyond a head's own dims, also where the page held something else before)."""
    T, eps, base = 23, 1e-5, 10000.0
    D = ops.attention_row_dim(dk, dv, dtype)
    g = torch.Generator(device="cuda").manual_seed(nh * dk + dv)
    extra = 8 if nh % 2 == 0 else 7      # columns that belong to something else (a gate) after the values; 7: rows that no vector access fits
    W = nh * dk + (nkv * (dk + dv) if write else 0) + extra
    proj = (torch.randn(T, W, device="cuda", generator=g) * 2).to(dtype)
    qw = 1 + 0.2 * torch.randn(dk, device="cuda", generator=g)
    kw = 1 + 0.2 * torch.randn(dk, device="cuda", generator=g)
    positions = torch.arange(100, 100 + T, dtype=torch.int32, device="cuda")
    cos = sin = None
    if rot:
        freq = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64).float().cuda()
        cos, sin = ops.rope_table(positions, freq)
    n_pages = -(-T // page) + 2
    cache = torch.full((n_pages, 2, nkv, page, D), 9.0, device="cuda", dtype=dtype)
    slots = (torch.randperm(n_pages * page, generator=torch.Generator().manual_seed(1))[:T]).to(torch.int32).cuda()
    q = ops.qk_norm_rope_write(proj, 0, nh * dk if write else -1, nh * dk + nkv * dk if write else -1, qw, kw if write else None,
                               eps, cos, sin, cache if write else None, slots if write else None, nh, nkv, dk, dv, D, rot, page)
    p64 = proj.double().cpu()
    want_q = MP.rotate_leading(MP.rms_norm(p64[:, :nh * dk].reshape(T, nh, dk), qw.double().cpu(), eps), positions.cpu(), rot, base)
    q = q.reshape(T, nh, D)
    # angles are fp32 products of a position near 100 and an fp32 frequency: 1e-5 of a radian off the 64-bit ones
    close(q[..., :dk], want_q, dtype, "queries", atol32=6e-5)
    assert float(q[..., dk:].abs().max()) == 0.0 if D > dk else True
    if not write:
        assert float((cache.float() - 9.0).abs().max()) == 0.0
        return
    want_k = MP.rotate_leading(MP.rms_norm(p64[:, nh * dk:nh * dk + nkv * dk].reshape(T, nkv, dk), kw.double().cpu(), eps),
                               positions.cpu(), rot, base)
    want_v = p64[:, nh * dk + nkv * dk:nh * dk + nkv * (dk + dv)].reshape(T, nkv, dv)
    flat = cache.permute(0, 3, 1, 2, 4).reshape(n_pages * page, 2, nkv, D)      # [slot, K|V, head, D]
    got = flat[slots.long()]
    close(got[:, 0, :, :dk], want_k, dtype, "keys", atol32=6e-5)
    close(got[:, 1, :, :dv], want_v, dtype, "values")
    assert float(got[:, 0, :, dk:].abs().sum()) == 0.0 and float(got[:, 1, :, dv:].abs().sum()) == 0.0
    untouched = torch.ones(n_pages * page, dtype=torch.bool)
    untouched[slots.long().cpu()] = False
    assert float((flat[untouched.cuda()].float() - 9.0).abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gates(ops, dtype):
    g = torch.Generator(device="cuda").manual_seed(4)
    T, nh, D, dv = 9, 5, 48, 40
    a = torch.randn(T, nh * D, device="cuda", generator=g).to(dtype)
    proj = (torch.randn(T, 11 + nh * dv, device="cuda", generator=g) * 3).to(dtype)
    want = a.double().reshape(T, nh, D)[..., :dv].reshape(T, nh * dv)
    close(ops.sigmoid_gate(a, D, None, 0, nh, dv), want, dtype, "narrowed")
    close(ops.sigmoid_gate(a, D, proj, 11, nh, dv), want * MP.sigmoid(proj.double()[:, 11:]), dtype, "gated")
    o = torch.randn(T, nh * dv, device="cuda", generator=g) * 5
    w = 1 + 0.1 * torch.randn(nh * dv, device="cuda", generator=g)
    want = MP.rms_norm(o.double(), w.double(), 1e-6)
    close(ops.rmsnorm_gate(o, w, 1e-6, None, 0, dtype), want, dtype, "row norm")
    close(ops.rmsnorm_gate(o, w, 1e-6, proj, 11, dtype), want * MP.sigmoid(proj.double()[:, 11:]), dtype, "row norm, gated")


# --------------------------------------------------------------------------- attention with a sink, every kernel
def plain_sink_attention_paged(q, cache, table, seq_of_token, positions, nh, nkv, D, scale, sink):
    """Every query over the keys 0..its position of its sequence, read through the block table; the softmax has
    exp(sink) more in its denominator."""
    page = cache.shape[3]
    out = torch.zeros_like(q, dtype=torch.float64)
    c = cache.double()
    for t in range(q.shape[0]):
        b, p = int(seq_of_token[t]), int(positions[t])
        pos = torch.arange(p + 1)
        pages = table[b].long()[pos // page]
        keys, vals = c[pages, 0, :, pos % page], c[pages, 1, :, pos % page]      # [keys, nkv, D]
        qt = q[t].double().reshape(nkv, nh // nkv, D)
        s = torch.einsum("grd,kgd->grk", qt, keys) * scale
        top = s.max(dim=-1, keepdim=True).values.clamp_min(sink)
        e = torch.exp(s - top)
        pr = e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink - top))
        out[t] = torch.einsum("grk,kgd->grd", pr, vals).reshape(-1)
    return out


@pytest.mark.parametrize("nh,nkv,D,page", [(4, 2, 64, 16), (6, 1, 128, 8), (5, 5, 32, 16), (8, 2, 64, 32)])
def test_sink_in_every_attention_kernel(ops, nh, nkv, D, page):
    """Prompt portions (deep in a context, whole, exactly 64 tokens) beside decoded tokens in one step, with the
    sink's term in every denominator: the dispatcher's choice of kernels, each prompt kernel alone, the split-KV
    kernel with one split, with a cluster of splits and with splits through scratch memory, and the exact kernel in
    both storage types.  One row's scores are all far below the sink (its output is next to nothing), one row's
    far key stands out, and the sum of a row's weights is below one by the sink's share."""
    from pyre_b200.engine.context import StepContext
    g = torch.Generator(device="cuda").manual_seed(D + page)
    ctx_lens, new = [450, 100, 64, 333, 77, 40, 1], [150, 100, 64, 1, 1, 20, 1]
    B = len(new)
    n_pages = sum(-(-c // page) for c in ctx_lens) + 3
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(2)).tolist()
    table = torch.full((B, max(-(-c // page) for c in ctx_lens)), -1, dtype=torch.int32)
    for s_, c in enumerate(ctx_lens):
        for lp in range(-(-c // page)):
            table[s_, lp] = perm.pop()
    cache = torch.randn(n_pages, 2, nkv, page, D, device="cuda", generator=g)
    seq_of_token = torch.tensor(sum(([s_] * n for s_, n in enumerate(new)), []), dtype=torch.int32)
    positions = torch.tensor(sum((list(range(c - n, c)) for c, n in zip(ctx_lens, new)), []), dtype=torch.int32)
    cu_host = np.concatenate([[0], np.cumsum(new)]).astype(np.int32)
    T = int(seq_of_token.shape[0])
    q = torch.randn(T, nh * D, device="cuda", generator=g) * 1.5
    scale = 0.9 * D ** -0.5
    far_row, low_row = 77, 200       # in the first and in the second sequence
    pg, off = int(table[0, 5 // page]), 5 % page
    cache[:, 0, 0] = cache[:, 0, 0].abs()                          # keys of head 0 are positive everywhere, so that ...
    q[low_row] = 0.0
    q[low_row, :D] = -40.0                                         # ... every score of this row's head 0 is far below 0
    cache[pg, 0, 0, off] = q[far_row, :D] * 2.0                    # key 5 of sequence 0 decides head 0 of this row
    cache16, q16 = cache.to(torch.bfloat16), q.to(torch.bfloat16)
    table_d, seq_d, pos_d, cu = table.cuda(), seq_of_token.cuda(), positions.cuda(), torch.from_numpy(cu_host).cuda()
    want = plain_sink_attention_paged(q16.cpu(), cache16.cpu(), table, seq_of_token, positions, nh, nkv, D, scale, 0.0)
    no_sink = plain_sink_attention_paged(q16.cpu(), cache16.cpu(), table, seq_of_token, positions, nh, nkv, D, scale, -1e30)
    assert (want - no_sink).abs().max() > 0.05, "the sink must matter in this test"
    assert want[low_row, :D].abs().max() < 1e-6 and no_sink[low_row, :D].abs().max() > 0.1

    def check(got, rows, what):
        assert torch.isfinite(got[rows]).all(), what
        err = (got[rows].double().cpu() - want[rows]).abs()
        bad = (err > 1.2e-2 + 1.6e-2 * want[rows].abs()).any(dim=1)
        assert not bad.any(), f"{what}: first wrong row {int(torch.where(bad)[0][0])}, max error {float(err.max()):.3e}"

    z = torch.zeros(T, dtype=torch.int32, device="cuda")
    ctx = StepContext(dtype=torch.bfloat16, device=torch.device("cuda"), num_tokens=T, num_seqs=B, num_logit_rows=0,
                      token_ids=z, positions=pos_d, seq_of_token=seq_d, cu_seqlens=cu, logit_rows=z[:0],
                      cu_seqlens_host=cu_host, start_pos_host=np.asarray([c - n for c, n in zip(ctx_lens, new)]))
    everything = slice(0, T)
    if D in ops.PREFILL_HEAD_DIMS or D <= ops.MMA_MAX_HEAD_DIM:
        got = ops.paged_attention_bf16(ctx, q16, cache16, table_d, nh, nkv, D, scale, None, sink=0.0)
        check(got, everything, "dispatch")
        v_far = cache16[pg, 1, 0, off].float()
        assert (got[far_row, :D].float() - v_far).abs().max() < 0.25 * v_far.abs().max() + 0.1
    if D in ops.PREFILL_HEAD_DIMS:
        out = torch.full_like(q16, 7.0)
        ops.attention_prefill(q16, cache16, table_d, cu, pos_d, B, 314, nh, nkv, D, scale, None, out, sink=0.0)
        check(out, slice(0, 314), "mma.sync prompt kernel")
        if page & (page - 1) == 0:
            for splits in (1, 3):
                out = torch.full_like(q16, 7.0)
                ops.attention_prefill_tc(q16, cache16, table_d, cu, pos_d, B, 314, nh, nkv, D, scale, None, out, 64, splits, sink=0.0)
                check(out, slice(0, 314), f"tcgen05 prompt kernel, {splits} share(s) of the keys")
    for splits, scratch in ((1, None), (4, None), (5, "scratch")):
        out = torch.full_like(q16, 7.0)
        sc = torch.empty(T * nh * splits * (D + 2), dtype=torch.float32, device="cuda") if scratch else None
        ops.paged_attention_mma(q16, cache16, table_d, cu, pos_d, B, nh, nkv, D, scale, None, splits, out=out, scratch=sc, sink=0.0)
        check(out, everything, f"split-KV kernel, {splits} split(s){' through scratch' if scratch else ''}")
    check(ops.paged_attention_generic(q16, cache16, table_d, seq_d, pos_d, nh, nkv, D, scale, None, sink=0.0), everything, "exact kernel, bf16 storage")
    got32 = ops.paged_attention_generic(q16.float(), cache16.float(), table_d, seq_d, pos_d, nh, nkv, D, scale, None, sink=0.0)
    torch.testing.assert_close(got32.double().cpu(), want, rtol=2e-5, atol=2e-6)
    # without a sink the kernels are what they were
    got = ops.paged_attention_generic(q16.float(), cache16.float(), table_d, seq_d, pos_d, nh, nkv, D, scale, None)
    torch.testing.assert_close(got.double().cpu(), no_sink, rtol=1e-4, atol=1e-5)      # scores near -300 in one row: fp32 rounds them by 3e-5
    ops.check_device_errors()


# --------------------------------------------------------------------------- linear attention over state slots
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hn,dk,dv,decay", [(3, 16, 24, [0.5, 0.9, 1.0]), (2, 64, 32, [0.999, 0.97]), (1, 20, 12, [0.8]),
                                            (2, 256, 48, [0.9995, 0.6]), (4, 128, 128, [0.99, 0.9, 0.5, 0.999])])
def test_linear_attention_over_state_slots(ops, dtype, Hn, dk, dv, decay):
    """Entries of unequal length in one launch, continued over three launches (a long portion, portions of 2 and 1
    tokens, single tokens) on slots that are not in order; the state starts at zero.  One query and one key far
    back are scaled so that this key's value decides an output hundreds of tokens later."""
    g = torch.Generator(device="cuda").manual_seed(dk * dv)
    lens = [300, 37, 1, 2]
    W = 5 + Hn * (2 * dk + dv)
    q_col, k_col, v_col = 5, 5 + Hn * dk, 5 + 2 * Hn * dk
    seqs = [(torch.randn(n, W, device="cuda", generator=g) * (1.0 if dk <= 64 else 0.5)) for n in lens]
    seqs[0][3, k_col:k_col + dk] = 6.0          # key 3 of head 0 ...
    seqs[0][290, q_col:q_col + dk] = 6.0        # ... meets query 290 of head 0
    seqs = [s.to(dtype) for s in seqs]
    d = torch.tensor(decay, dtype=torch.float32, device="cuda")
    want = []
    for s in seqs:
        x = s.double().cpu()
        n = x.shape[0]
        rb = (lambda z: z.to(torch.bfloat16).double()) if dtype == torch.bfloat16 else (lambda z: z)      # q, k, v are activations
        qq, kk = rb(MP.silu(x[:, q_col:q_col + Hn * dk])).reshape(n, Hn, dk), rb(MP.silu(x[:, k_col:k_col + Hn * dk])).reshape(n, Hn, dk)
        vv = rb(MP.silu(x[:, v_col:v_col + Hn * dv])).reshape(n, Hn, dv)
        want.append(MP.decayed_linear_attention(qq, kk, vv, d.double().cpu()).reshape(n, Hn * dv))
    state = torch.full((6, Hn, dk, dv), float("nan"), device="cuda")
    slot_of = [4, 0, 5, 2]
    state[slot_of] = 0.0
    got = [[] for _ in lens]
    cuts = [[0, 170, 299, 300], [0, 35, 36, 37], [0, 1, 1, 1], [0, 0, 2, 2]]
    for step in range(3):
        rows, slots, cu, who = [], [], [0], []
        for b, s in enumerate(seqs):
            lo, hi = cuts[b][step], cuts[b][step + 1]
            if hi > lo:
                rows.append(s[lo:hi]); slots.append(slot_of[b]); cu.append(cu[-1] + hi - lo); who.append(b)
        out = ops.linear_attention(torch.cat(rows).contiguous(), q_col, k_col, v_col, state, torch.tensor(slots, dtype=torch.int32, device="cuda"),
                                   torch.tensor(cu, dtype=torch.int32, device="cuda"), d, Hn, dk, dv, "silu")
        for i, b in enumerate(who):
            got[b].append(out[cu[i]:cu[i + 1]])
    assert torch.isnan(state[[1, 3]]).all(), "slots of no entry were touched"
    for b in range(len(lens)):
        g_b, w_b = torch.cat(got[b]).double().cpu(), want[b]
        scale = float(w_b.abs().max())
        assert (g_b - w_b).abs().max() <= 2e-5 * scale + 1e-6, f"entry {b}: {(g_b - w_b).abs().max():.3e} of {scale:.3e}"


@pytest.mark.parametrize("Hn,dk,dv,decay", [(3, 64, 32, [0.5, 0.97, 1.0]), (2, 128, 64, [0.999, 0.9]), (1, 128, 128, [0.99]),
                                            (4, 64, 96, [0.3, 0.8, 0.995, 0.9999])])
def test_linear_attention_on_the_tensor_cores(ops, Hn, dk, dv, decay):
    """Prompt portions of 32 tokens and more take the chunked kernel (chunks of 64 tokens; a portion of exactly one
    chunk, one token more, a ragged end), shorter entries beside them the token-by-token kernel, and a request goes
    from one to the other and back between steps with its state; the result is that of the recurrence on the same
    bf16-rounded q, k, v up to the rounding of sums.  A far key decides an output 287 tokens on."""
    g = torch.Generator(device="cuda").manual_seed(dk + dv)
    lens = [300, 37, 64, 65, 2, 131]
    W = 8 + Hn * (2 * dk + dv)
    q_col, k_col, v_col = 8, 8 + Hn * dk, 8 + 2 * Hn * dk
    assert ops.linear_chunks_ok(W, q_col, k_col, v_col, dk, dv)
    seqs = [torch.randn(n, W, device="cuda", generator=g) * (1.0 if dk <= 64 else 0.6) for n in lens]
    seqs[0][3, k_col:k_col + dk] = 6.0
    seqs[0][290, q_col:q_col + dk] = 6.0
    seqs = [s.to(torch.bfloat16) for s in seqs]
    d = torch.tensor(decay, dtype=torch.float32, device="cuda")
    rb = lambda x: x.to(torch.bfloat16).double()
    want = []
    for s in seqs:
        x = s.double().cpu()
        n = x.shape[0]
        qq, kk = rb(MP.silu(x[:, q_col:q_col + Hn * dk])).reshape(n, Hn, dk), rb(MP.silu(x[:, k_col:k_col + Hn * dk])).reshape(n, Hn, dk)
        vv = rb(MP.silu(x[:, v_col:v_col + Hn * dv])).reshape(n, Hn, dv)
        want.append(MP.decayed_linear_attention(qq, kk, vv, d.double().cpu()).reshape(n, Hn * dv))
    state = torch.full((8, Hn, dk, dv), float("nan"), device="cuda")
    slot_of = [4, 0, 5, 2, 7, 1]
    state[slot_of] = 0.0
    got = [[] for _ in lens]
    # entry 0: 170 tokens (chunks), then 31 (token by token), then 99 (chunks); entry 5: 1 token, then 130 (chunks)
    cuts = [[0, 170, 201, 300], [0, 37, 37, 37], [0, 0, 64, 64], [0, 65, 65, 65], [0, 0, 2, 2], [0, 1, 131, 131]]
    for step in range(3):
        rows, slots, cu, who = [], [], [0], []
        for b, s in enumerate(seqs):
            lo, hi = cuts[b][step], cuts[b][step + 1]
            if hi > lo:
                rows.append(s[lo:hi]); slots.append(slot_of[b]); cu.append(cu[-1] + hi - lo); who.append(b)
        out = ops.linear_attention(torch.cat(rows).contiguous(), q_col, k_col, v_col, state, torch.tensor(slots, dtype=torch.int32, device="cuda"),
                                   torch.tensor(cu, dtype=torch.int32, device="cuda"), d, Hn, dk, dv, "silu", lens=np.diff(np.asarray(cu)))
        for i, b in enumerate(who):
            got[b].append(out[cu[i]:cu[i + 1]])
    assert torch.isnan(state[[3, 6]]).all(), "slots of no entry were touched"
    assert torch.isfinite(state[slot_of]).all()
    for b in range(len(lens)):
        g_b, w_b = torch.cat(got[b]).double().cpu(), want[b]
        assert torch.isfinite(g_b).all(), f"entry {b}"
        err = (g_b - w_b).abs().max(dim=1).values
        scale = w_b.abs().max(dim=1).values.clamp_min(float(w_b.abs().mean()))
        bad = err > 3e-4 * scale + 1e-5
        assert not bad.any(), f"entry {b}: first wrong token {int(torch.where(bad)[0][0])} of {lens[b]}: {float(err[bad][0]):.3e} of {float(scale[bad][0]):.3e}"
    ops.check_device_errors()


# --------------------------------------------------------------------------- the engine against the plain model
LENGTHS = {"P": [1, 2, 17, 33, 70, 130], "Q": [3, 40, 63, 64, 65, 200], "R": [5, 31, 97, 150], "S": [2, 47, 129, 260]}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for n, (name, raw) in enumerate(MH.MODO.items()):
        d = tmp_path_factory.mktemp(f"modovik_{name}")
        MH.make_modovik_dir(d, raw, seed=500 + n)
        reqs = {f"{name}{i}": H.random_ids(raw["vocab"], L, seed=13 * n + i) for i, L in enumerate(LENGTHS[name])}
        plain = {rid: MH.plain_logits(d, ids) for rid, ids in reqs.items()}
        sq, cnt = 0.0, 0
        for rid, ids in reqs.items():
            e = MH.plain_logits(d, ids, lowp=True) - plain[rid]
            sq, cnt = sq + float((e ** 2).sum()), cnt + e.size
        out[name] = (d, reqs, plain, math.sqrt(sq / cnt))
    return out


def run(models, name, dtype, steps, what, want=None):
    d, reqs, plain, lowp_rms = models[name]
    got = H.run_trace_in_process(d, dtype, steps, H.max_live_tokens(steps), MH.MODO_PAGE_SIZE[name])
    MH.compare(got, want or plain, dtype, what, lowp_rms)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q", "R", "S"])
def test_whole_prompts(models, name, dtype):
    run(models, name, dtype, H.trace_whole(models[name][1]), "whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q", "R", "S"])
def test_prefill_then_token_by_token(models, name, dtype):
    steps = []
    for k, (rid, ids) in enumerate(models[name][1].items()):
        # most of it in one step and the rest one by one; every third request one by one from its first token
        steps += H.trace_decode_tail(rid, ids, len(ids) if k % 3 == 2 else 32, first_step=len(steps))
    run(models, name, dtype, steps, "decode")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q", "R", "S"])
def test_portions_down_to_two_tokens(models, name, dtype):
    steps = []
    for k, (rid, ids) in enumerate(models[name][1].items()):
        sizes = [[2, 9, 3, 17, 2, 31], [5, 2, 16, 8, 64], [24, 2, 2, 7, 1, 70]][k % 3]
        steps += H.trace_portions(rid, ids, sizes, first_step=len(steps))
    run(models, name, dtype, steps, "portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q", "R", "S"])
def test_mixed_batches_reuse_pages_and_slots(models, name, dtype):
    """Every request twice under other names, at most four alive: later ones get the pages (filled with NaN when
    they were given back) and the state slots that earlier ones held, and must come out as each alone."""
    d, reqs, plain, _ = models[name]
    many = {f"{rid}r{rep}": ids for rep in range(2) for rid, ids in reqs.items()}
    steps = H.trace_mixed(many, seed=21, max_live=4, portion=(2, 40))
    run(models, name, dtype, steps, "mixed", {f"{rid}r{rep}": plain[rid] for rep in range(2) for rid in reqs})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_state_slots_are_zeroed_for_the_next_request(models, dtype):
    """Four slots only: the fifth request begins in a slot whose last owner left a state behind."""
    from pyre_b200.engine import replay as rp
    from pyre_b200.models.model import load_model
    d, reqs, plain, lowp_rms = models["P"]
    model, _ = load_model(d, "cuda:0", dtype)
    cache, stepper = rp.runtime_for_model(model, 4096, 16, max_requests=4)
    from pyre_b200.engine.step import StepEntry
    ids = reqs["P4"]
    got = {}
    for rep in range(6):
        rid = f"again{rep}"
        cache.begin(rid)
        got[rid] = stepper.step([StepEntry(rid, ids, list(range(len(ids))))]).cpu().numpy()
        assert cache.state.slot_of[rid] < 4
        cache.end(rid)
    MH.compare(got, {rid: plain["P4"] for rid in got}, dtype, "slot reuse", lowp_rms)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q"])
def test_long_decoding(models, tmp_path, name, dtype):
    """400 tokens, the last 330 one by one (captured decode steps), two requests side by side."""
    d, _reqs, _plain, lowp_rms = models[name]
    vocab = MH.MODO[name]["vocab"]
    reqs = {f"long{i}": H.random_ids(vocab, n, seed=90 + i) for i, n in enumerate([400, 370])}
    steps = [{"step": 0, "entries": [{"id": r, "tokens": ids[:70 - 30 * i], "want": [0]} for i, (r, ids) in enumerate(reqs.items())], "end": []}]
    at = {r: 70 - 30 * i for i, r in enumerate(reqs)}
    while any(at[r] < len(reqs[r]) for r in reqs):
        entries = [{"id": r, "tokens": [reqs[r][at[r]]], "want": [0]} for r in reqs if at[r] < len(reqs[r])]
        for e in entries:
            at[e["id"]] += 1
        steps.append({"step": len(steps), "entries": entries, "end": [e["id"] for e in entries if at[e["id"]] == len(reqs[e["id"]])]})
    got = H.run_trace_in_process(d, dtype, steps, H.max_live_tokens(steps), MH.MODO_PAGE_SIZE[name])
    want = {}
    for i, (r, ids) in enumerate(reqs.items()):
        full = MH.plain_logits(d, ids)
        want[r] = np.concatenate([full[:1], full[70 - 30 * i:]])
    MH.compare(got, want, dtype, "long decoding", lowp_rms)


@pytest.mark.parametrize("name", ["P", "S"])
def test_greedy_generation_through_the_engine(models, name):
    """``Engine.generate`` (scheduler, portions of prompts, captured decode steps, sampler) gives the tokens that
    the plain implementation's argmax gives, in 32-bit; a cache too small for all requests at once makes the
    scheduler preempt and recompute, state included."""
    from pyre_b200.engine.engine import Engine
    from pyre_b200.sampling import SamplingParams
    d, _reqs, _plain, _ = models[name]
    raw = MH.MODO[name]
    prompts = [H.random_ids(raw["vocab"], n, seed=40 + n) for n in (15, 16, 3, 30)]
    new = 20
    # three requests of one page each are admitted; two tokens on, each wants a second page and five are not enough
    engine = Engine(str(d), dtype="float32", page_size=16, num_pages=5, max_num_seqs=3, max_num_batched_tokens=32, prefill_chunk=20)
    outs = engine.generate(prompts, SamplingParams(max_new_tokens=new, return_logits=True))
    for p, o in zip(prompts, outs):
        ids = list(p)
        for k in range(new):
            logits = MH.plain_logits(d, ids)[-1]
            top2 = np.sort(logits)[-2:]
            np.testing.assert_allclose(o.logits[k], logits, rtol=2e-4, atol=3e-5)
            if top2[1] - top2[0] > 1e-4:
                assert o.token_ids[k] == int(logits.argmax()), f"token {k} of a prompt of {len(p)}"
            ids.append(o.token_ids[k])
    assert engine.stats()["preempted"] > 0, "the cache was meant to be too small for all requests at once"
    assert json.dumps(engine.stats())
