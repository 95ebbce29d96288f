"""Each CUDA kernel alone against a plain float32 reference, at sizes other than the engine's
test models use (odd widths, head sizes in steps of 16, groups of 1 to 8, vocabularies that
are no power of two)."""
import math
import os
import random

import pytest
import torch

from tests.plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, scale=1.0):
    return (2e-5 if dtype == torch.float32 else 2e-2) * scale


def dev(t, dtype=None):
    return t.to(device="cuda", dtype=dtype or t.dtype).contiguous()


@pytest.fixture(scope="module")
def ops():
    from llmgen_b200.kernels import ops as o
    return o


# ------------------------------------------------------------------ elementwise
@pytest.mark.parametrize("dtype", DTYPES)
def test_embed_rows(ops, dtype):
    torch.manual_seed(0)
    V, H = 100, 72
    table = torch.randn(V, H).to(dtype)
    ids = torch.tensor([3, 99, 0, 57, 3], dtype=torch.int32)
    out = torch.empty(5, H, dtype=torch.float32, device="cuda")
    bad = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.embed_rows(out, dev(table), dev(ids), bad)
    assert torch.equal(out.cpu(), plain.embedding(ids.tolist(), table.float()))
    assert int(bad.item()) == 0
    ops.embed_rows(out, dev(table), dev(torch.tensor([1, 100, -1, 2, 5], dtype=torch.int32)), bad)
    assert int(bad.item()) == 2 and float(out[1].abs().sum()) == 0.0 and float(out[2].abs().sum()) == 0.0
    assert torch.equal(out[3].cpu(), table[2].float())
    # rows whose id is the one the step before sampled (still on the device), beside rows the host names
    sampled = dev(torch.tensor([7, 8, 9], dtype=torch.int32))
    ids_from = dev(torch.tensor([-1, 2, 0, -1, 1], dtype=torch.int32))
    bad.zero_()
    ops.embed_rows(out, dev(table), dev(ids), bad, ids_from=ids_from, sampled=sampled)
    assert torch.equal(out.cpu(), plain.embedding([3, 9, 7, 57, 8], table.float())) and int(bad.item()) == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H", [100, 1030, 1032, 5120, 8200])
def test_add_rmsnorm(ops, dtype, H):
    torch.manual_seed(1)
    n, eps = 7, 3e-5
    resid = torch.randn(n, H) * 2
    delta = torch.randn(n, H).to(dtype)
    w = 1 + 0.2 * torch.randn(H)
    r = dev(resid)
    out = torch.empty(n, H, dtype=dtype, device="cuda")
    ops.add_rmsnorm(r, dev(delta), dev(w), out, eps, 0.0)
    summed = resid + delta.float()
    assert torch.allclose(r.cpu(), summed, atol=1e-6)          # the sum stays float32
    ref = plain.rmsnorm(summed, w, eps)
    assert float((out.float().cpu() - ref).abs().max()) < tol(dtype, 6)
    # no delta, a weight offset, gathered rows, residual untouched
    rows = torch.tensor([5, 0, 5], dtype=torch.int32)
    out2 = torch.empty(3, H, dtype=dtype, device="cuda")
    before = r.clone()
    ops.add_rmsnorm(r, None, dev(w), out2, eps, 1.0, rows=dev(rows))
    assert torch.equal(r, before)
    ref2 = plain.rmsnorm(summed[rows.long()], w, eps, weight_offset=1.0)
    assert float((out2.float().cpu() - ref2).abs().max()) < tol(dtype, 10)
    # gathered rows with a pending delta
    r3 = dev(resid)
    ops.add_rmsnorm(r3, dev(delta), dev(w), out2, eps, 0.0, rows=dev(rows))
    assert torch.equal(r3.cpu(), resid)
    assert float((out2.float().cpu() - ref[rows.long()]).abs().max()) < tol(dtype, 6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,H", [(603, 1024), (512, 80), (700, 1536), (515, 2048), (513, 132)])
def test_add_rmsnorm_of_many_rows(ops, dtype, n, H):
    """A prompt's rows: the variant with a warp per row (512 rows and more, widths up to 2,048), with
    a delta, without one, and with the residual left as it was."""
    torch.manual_seed(3)
    eps = 2e-6
    resid = torch.randn(n, H) * 2
    resid[n - 1] *= 40.0                                        # a last row that stands out: no row is skipped or swapped
    delta = torch.randn(n, H).to(dtype)
    w = 1 + 0.2 * torch.randn(H)
    r = dev(resid)
    out = torch.empty(n, H, dtype=dtype, device="cuda")
    ops.add_rmsnorm(r, dev(delta), dev(w), out, eps, 0.0)
    summed = resid + delta.float()
    assert torch.allclose(r.cpu(), summed, atol=1e-5)
    assert float((out.float().cpu() - plain.rmsnorm(summed, w, eps)).abs().max()) < tol(dtype, 6)
    before = r.clone()
    ops.add_rmsnorm(r, None, dev(w), out, eps, 1.0)
    assert torch.equal(r, before)
    assert float((out.float().cpu() - plain.rmsnorm(summed, w, eps, weight_offset=1.0)).abs().max()) < tol(dtype, 10)
    ops.add_rmsnorm(r, dev(delta), dev(w), out, eps, 0.0, write_resid=False)
    assert torch.equal(r, before)
    assert float((out.float().cpu() - plain.rmsnorm(summed + delta.float(), w, eps)).abs().max()) < tol(dtype, 6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("F", [50, 64, 176])
def test_silu_mul(ops, dtype, F):
    torch.manual_seed(2)
    x = (torch.randn(9, 2 * F) * 3).to(dtype)
    out = torch.empty(9, F, dtype=dtype, device="cuda")
    ops.silu_mul(out, dev(x))
    g, u = x.float()[:, :F], x.float()[:, F:]
    ref = g / (1 + torch.exp(-g)) * u
    assert torch.allclose(out.float().cpu(), ref, rtol=1e-5 if dtype == torch.float32 else 1e-2, atol=tol(dtype))
    if F % 16 == 0:        # gate and up alternating in groups of 16 columns
        mixed = torch.stack([x[:, :F].reshape(9, F // 16, 16), x[:, F:].reshape(9, F // 16, 16)], dim=2).reshape(9, 2 * F)
        out2 = torch.empty(9, F, dtype=dtype, device="cuda")
        ops.silu_mul(out2, dev(mixed), group=16)
        assert torch.equal(out2, out)


# ------------------------------------------------------------------ attn_prep
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,hd,rot", [(5, 1, 48, 48), (4, 2, 16, 16), (3, 3, 64, 32), (16, 8, 128, 128), (2, 1, 256, 256)])
def test_attn_prep(ops, dtype, nq, nkv, hd, rot):
    torch.manual_seed(3)
    T, page, pages, eps = 6, 8, 5, 1e-5
    qkv = torch.randn(T, (nq + 2 * nkv) * hd).to(dtype)
    positions = [3, 17, 0, 42, 9, 41]
    slots = [5, 17, -1, 0, 39, 16]                      # page * 8 + offset; -1: do not store
    qg, kg = 1 + 0.3 * torch.randn(hd), 1 + 0.3 * torch.randn(hd)
    cos64, sin64 = plain.rope_tables(64, rot, 10000.0)
    kc = torch.full((pages, nkv, page, hd), 7.0, dtype=dtype, device="cuda")
    vc = torch.full((pages, nkv, page, hd), 7.0, dtype=dtype, device="cuda")
    x = dev(qkv)
    ops.attn_prep(x, kc, vc, dev(torch.tensor(positions, dtype=torch.int32)), dev(torch.tensor(slots, dtype=torch.int32)),
                  dev(cos64.float()), dev(sin64.float()), dev(qg), dev(kg), nq, nkv, hd, rot, page, eps)
    f = qkv.float()
    q = f[:, :nq * hd].view(T, nq, hd)
    k = f[:, nq * hd:(nq + nkv) * hd].view(T, nkv, hd)
    v = f[:, (nq + nkv) * hd:].view(T, nkv, hd)
    q_ref = plain.apply_rope(plain.rmsnorm(q, qg, eps), positions, cos64, sin64, rot)
    k_ref = plain.apply_rope(plain.rmsnorm(k, kg, eps), positions, cos64, sin64, rot)
    got_q = x.float().cpu()[:, :nq * hd].view(T, nq, hd)
    assert float((got_q - q_ref).abs().max()) < tol(dtype, 6)
    kc_ref = torch.full((pages, nkv, page, hd), 7.0)
    vc_ref = torch.full((pages, nkv, page, hd), 7.0)
    for t, s in enumerate(slots):
        if s >= 0:
            kc_ref[s // page, :, s % page] = k_ref[t]
            vc_ref[s // page, :, s % page] = v[t]
    assert float((kc.float().cpu() - kc_ref).abs().max()) < tol(dtype, 6)
    assert torch.equal(vc.float().cpu(), vc_ref)                       # values are copied bit for bit
    # the k and v columns of the packed rows are left as they were
    assert torch.equal(x.cpu()[:, nq * hd:], qkv[:, nq * hd:])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,hd", [(4, 2, 64), (16, 8, 128), (3, 1, 256), (5, 2, 32), (2, 2, 48)])
@pytest.mark.parametrize("T", [32, 77, 300])
@pytest.mark.parametrize("by_token", [True, False])
def test_attn_prep_on_prompts(ops, dtype, nq, nkv, hd, T, by_token):
    """Many rows: the paths with 16-byte accesses (head sizes they take; a warp on several heads of a
    token, or a row at a time) and the general one agree with the plain functions; slots include -1
    and a page's last place; q lands in a buffer of its own."""
    ops.attn_prep_set_by_token(by_token)
    try:
        _attn_prep_on_prompts(ops, dtype, nq, nkv, hd, T)
    finally:
        ops.attn_prep_set_by_token(True)


def _attn_prep_on_prompts(ops, dtype, nq, nkv, hd, T):
    torch.manual_seed(4)
    page, eps = 16, 1e-6
    pages = (T + page - 1) // page + 1
    qkv = torch.randn(T, (nq + 2 * nkv) * hd).to(dtype)
    positions = [(7 * t) % 200 for t in range(T)]
    perm = torch.randperm(pages * page)[:T].tolist()
    slots = [-1 if t % 11 == 5 else perm[t] for t in range(T)]
    qg, kg = 1 + 0.3 * torch.randn(hd), 1 + 0.3 * torch.randn(hd)
    cos, sin = plain.rope_tables(200, hd, 10000.0)
    kc = torch.full((pages, nkv, page, hd), 7.0, dtype=dtype, device="cuda")
    vc = torch.full((pages, nkv, page, hd), 7.0, dtype=dtype, device="cuda")
    x = dev(qkv)
    q_out = torch.full((T, nq * hd), 9.0, dtype=dtype, device="cuda")
    ops.attn_prep(x, kc, vc, dev(torch.tensor(positions, dtype=torch.int32)), dev(torch.tensor(slots, dtype=torch.int32)),
                  dev(cos.float()), dev(sin.float()), dev(qg), dev(kg), nq, nkv, hd, hd, page, eps, q_out=q_out)
    f = qkv.float()
    q = f[:, :nq * hd].view(T, nq, hd)
    k = f[:, nq * hd:(nq + nkv) * hd].view(T, nkv, hd)
    v = f[:, (nq + nkv) * hd:].view(T, nkv, hd)
    q_ref = plain.apply_rope(plain.rmsnorm(q, qg, eps), positions, cos, sin, hd)
    k_ref = plain.apply_rope(plain.rmsnorm(k, kg, eps), positions, cos, sin, hd)
    assert float((q_out.float().cpu().view(T, nq, hd) - q_ref).abs().max()) < tol(dtype, 6)
    kc_ref = torch.full((pages, nkv, page, hd), 7.0)
    vc_ref = torch.full((pages, nkv, page, hd), 7.0)
    for t, s in enumerate(slots):
        if s >= 0:
            kc_ref[s // page, :, s % page] = k_ref[t]
            vc_ref[s // page, :, s % page] = v[t]
    assert float((kc.float().cpu() - kc_ref).abs().max()) < tol(dtype, 6)
    assert torch.equal(vc.float().cpu(), vc_ref)
    assert torch.equal(x.cpu(), qkv)                                   # the packed rows are left as they were


@pytest.mark.parametrize("dtype", DTYPES)
def test_attn_prep_without_norm_or_rope_and_q_only(ops, dtype):
    torch.manual_seed(4)
    T, nq, nkv, hd = 3, 2, 1, 32
    qkv = torch.randn(T, (nq + 2 * nkv) * hd).to(dtype)
    kc = torch.zeros(2, nkv, 4, hd, dtype=dtype, device="cuda")
    vc = torch.zeros_like(kc)
    x = dev(qkv)
    ops.attn_prep(x, kc, vc, None, dev(torch.tensor([0, 5, 2], dtype=torch.int32)), None, None, None, None,
                  nq, nkv, hd, 0, 4, 0.0)
    assert torch.equal(x.cpu(), qkv)
    assert torch.equal(kc.cpu()[1, 0, 1], qkv[1, nq * hd:(nq + 1) * hd])
    # a layer that reads another layer's cache: only q heads are present, nothing is stored
    q_only = dev(qkv[:, :nq * hd].contiguous())
    kc.zero_()
    g = 1 + 0.1 * torch.randn(hd)
    ops.attn_prep(q_only, kc, vc, None, dev(torch.tensor([0, 5, 2], dtype=torch.int32)), None, None, dev(g), dev(g),
                  nq, 0, hd, 0, 4, 1e-6)
    assert float(kc.abs().sum()) == 0.0
    ref = plain.rmsnorm(qkv.float()[:, :nq * hd].view(T, nq, hd), g, 1e-6)
    assert float((q_only.float().cpu().view(T, nq, hd) - ref).abs().max()) < tol(dtype, 6)


def test_attn_prep_refuses_what_it_cannot_do(ops):
    x = torch.zeros(1, 3 * 18, dtype=torch.float32, device="cuda")
    with pytest.raises(ops.KernelError, match="head_dim"):
        ops.attn_prep(x, None, None, None, None, None, None, None, None, 1, 1, 17, 0, 4, 0.0)
    with pytest.raises(ops.KernelError, match="CUDA device"):
        ops.attn_prep(torch.zeros(1, 48), None, None, None, None, None, None, None, None, 1, 1, 16, 0, 4, 0.0)
    # a pairing or a per-head norm that no kernel implements is refused by name, not computed as another
    x16 = torch.zeros(1, 48, dtype=torch.float32, device="cuda")
    with pytest.raises(ops.KernelError, match="pairing"):
        ops.attn_prep(x16, None, None, None, None, None, None, None, None, 1, 1, 16, 0, 4, 0.0, pairing="interleaved")
    with pytest.raises(ops.KernelError, match="pairing"):
        ops.attn_prep(x16, None, None, None, None, None, None, None, None, 1, 1, 16, 0, 4, 0.0, pairing="spiral")
    with pytest.raises(ops.KernelError, match="normalises heads"):
        ops.attn_prep(x16, None, None, None, None, None, None, None, None, 1, 1, 16, 0, 4, 0.0, head_norm="layernorm")


# ------------------------------------------------------------------ matrix products
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M", [1, 2, 3, 4, 8, 33, 70])
def test_gemm_simt(ops, dtype, M):
    torch.manual_seed(5)
    N, K = 130, 77
    a = torch.randn(M, K).to(dtype)
    w = (torch.randn(N, K) * 0.2).to(dtype)
    out = torch.empty(M, N, dtype=dtype, device="cuda")
    ops.gemm_simt(out, dev(a), dev(w))
    ref = a.double() @ w.double().t()
    assert float((out.double().cpu() - ref).abs().max()) < tol(dtype, 4)
    if dtype == torch.bfloat16:                     # float32 output of a bfloat16 product
        out32 = torch.empty(M, N, dtype=torch.float32, device="cuda")
        ops.gemm_simt(out32, dev(a), dev(w))
        assert float((out32.double().cpu() - ref).abs().max()) < 1e-4
    # strided operands and accumulate
    big = torch.zeros(M, N + 6, dtype=dtype, device="cuda")
    view = big[:, 3:3 + N]
    ops.gemm_simt(view, dev(a), dev(w))
    ops.gemm_simt(view, dev(a), dev(w), accumulate=True)
    assert float((view.double().cpu() - 2 * ref).abs().max()) < tol(dtype, 12)
    assert float(big[:, :3].abs().sum()) == 0.0 and float(big[:, 3 + N:].abs().sum()) == 0.0


def test_gemm_simt_row_does_not_depend_on_the_batch(ops):
    """float32: a row's result is bit-identical whatever else is in the batch."""
    torch.manual_seed(6)
    a = dev(torch.randn(70, 333))
    w = dev(torch.randn(50, 333))
    full = torch.empty(70, 50, device="cuda")
    ops.gemm_simt(full, a, w)
    for rows in ([0], [69], list(range(10, 27))):
        part = torch.empty(len(rows), 50, device="cuda")
        ops.gemm_simt(part, a[rows].contiguous(), w)
        assert torch.equal(part, full[rows])


@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (5, 72, 136), (33, 384, 512), (128, 128, 64), (200, 1000, 1032),
                                   (257, 4096, 1024), (64, 130, 2048), (2048, 1024, 3072), (300, 50, 40)])
@pytest.mark.parametrize("out_dtype", DTYPES)
def test_gemm_tc(ops, M, N, K, out_dtype):
    """The tcgen05 product against a float64 reference of the same bfloat16 operands: every tile
    width, tails in M, N and K, float32 and bfloat16 results."""
    torch.manual_seed(50 + M)
    a = torch.randn(M, K).to(torch.bfloat16)
    w = (torch.randn(N, K) * 0.5).to(torch.bfloat16)
    # one entry that only the last k-slice sees, and one that only the last rows see
    a[M - 1, K - 1] = 8.0
    w[N - 1, K - 1] = 8.0
    out = torch.full((M, N), 7.0, dtype=out_dtype, device="cuda")
    ops.gemm_tc(out, dev(a), dev(w))
    torch.cuda.synchronize()
    ops.check_tc_errors(out.device)
    ref = a.double() @ w.double().t()
    scale = float(ref.abs().max())
    err = float((out.double().cpu() - ref).abs().max())
    assert err < (2e-5 if out_dtype == torch.float32 else 6e-3) * scale, (err, scale)
    # the same result inside a wider array with 16-byte aligned rows (where TMA stores are possible): what lies
    # around it is left alone, whatever N (a TMA store clips in units of 16 bytes, so other widths must not take it)
    buf = torch.full((M + 1, N + 24 - N % 8), 7.0, dtype=out_dtype, device="cuda")
    ops.gemm_tc(buf[:M, :N], dev(a), dev(w))
    torch.cuda.synchronize()
    assert torch.equal(buf[:M, :N], out)
    assert bool((buf[M] == 7.0).all()) and bool((buf[:, N:] == 7.0).all())


@pytest.mark.parametrize("M,N,K", [(8, 4096, 1024), (8, 1024, 2048), (8, 1024, 3072), (1, 6144, 1024), (3, 72, 136), (7, 1000, 1032),
                                   (5, 16, 8), (8, 130, 3072), (2, 48, 40), (4, 100, 520)])
def test_gemm_rows8(ops, M, N, K):
    """The product for up to 8 rows (W straight from global memory into mma.sync): its float32 slices add up to the
    product (float64 reference of the same bfloat16 operands); tails in N (no multiple of 16), in K (no multiple of
    32, slices that do not divide it), every M from 1 to 8; values that only the last k, the last row of W and each
    half of an MMA's 16 rows see; strided operands; refusals."""
    torch.manual_seed(80 + M + N)
    a = torch.randn(M, K + 8).to(torch.bfloat16)[:, :K]              # rows 16-byte aligned, not contiguous
    w = (torch.randn(N, K) * 0.5).to(torch.bfloat16)
    a[M - 1, K - 1] = 8.0
    w[N - 1, K - 1] = 8.0
    w[min(N - 1, 9), 0] = -6.0
    ad, wd = dev(a.contiguous())[:, :], dev(w)
    big = torch.zeros(M, K + 8, dtype=torch.bfloat16, device="cuda")
    big[:, :K] = ad
    ad = big[:, :K]
    assert ops.gemm_rows8_usable(ad, wd)
    slices = ops.gemm_rows8_slices(N, K)
    assert 1 <= slices <= 8
    out = torch.full((slices + 1, M, N), 7.0, dtype=torch.float32, device="cuda")
    ops.gemm_rows8(out[:slices], ad, wd)
    torch.cuda.synchronize()
    assert bool((out[slices] == 7.0).all())
    ref = a.double() @ w.double().t()
    scale = float(ref.abs().max())
    err = float((out[:slices].double().sum(0).cpu() - ref).abs().max())
    assert err < 2e-5 * scale, (err, scale)
    if K > 32 * 12:          # more than one slice: each holds its own columns of K only
        assert slices > 1 and float(out[0].abs().max()) > 0 and float((out[0] - out[:slices].sum(0)).abs().max()) > 0
    # 9 rows, a K of no whole 16-byte pieces, a K beyond 8 slices: refused
    assert not ops.gemm_rows8_usable(torch.zeros(9, K, dtype=torch.bfloat16, device="cuda"), wd)
    assert not ops.gemm_rows8_usable(torch.zeros(2, 3080, dtype=torch.bfloat16, device="cuda"), torch.zeros(16, 3080, dtype=torch.bfloat16, device="cuda"))
    assert not ops.gemm_rows8_usable(torch.zeros(2, 36, dtype=torch.bfloat16, device="cuda")[:, :34], torch.zeros(16, 34, dtype=torch.bfloat16, device="cuda"))


@pytest.mark.parametrize("M,F,K", [(8, 3072, 1024), (1, 3072, 1024), (4, 48, 128), (3, 176, 264), (7, 16, 8), (5, 1024, 1536), (2, 80, 1000)])
def test_gemm_rows8_gated(ops, M, F, K):
    """The gated form: silu(gate) * up of up to 8 rows against a float64 reference, W's rows interleaved in groups of
    16, every share of K that four warps take (also none for the last warps), F no multiple of the block's 16 columns
    beyond it; the surroundings of the result are left alone; a K that the warps' registers cannot hold is refused."""
    from llmgen_b200.parts.mlp import interleave_gate_up
    torch.manual_seed(190 + M + F)
    a = torch.randn(M, K).to(torch.bfloat16)
    wg = (torch.randn(F, K) * 0.1).to(torch.bfloat16)
    wu = (torch.randn(F, K) * 0.1).to(torch.bfloat16)
    a[M - 1, K - 1] = 4.0
    wg[F - 1, K - 1] = 2.0
    wu[min(F - 1, 9), 0] = -3.0
    w = dev(interleave_gate_up(wg, wu))
    assert ops.gemm_rows8_gated_usable(dev(a), w)
    buf = torch.full((M + 1, F + 8), 7.0, dtype=torch.bfloat16, device="cuda")
    ops.gemm_rows8_gated(buf[:M, :F], dev(a), w)
    torch.cuda.synchronize()
    g = a.double() @ wg.double().t()
    u = a.double() @ wu.double().t()
    ref = g / (1 + torch.exp(-g)) * u
    assert float((buf[:M, :F].double().cpu() - ref).abs().max()) < 8e-3 * max(1.0, float(ref.abs().max()))
    assert bool((buf[M] == 7.0).all()) and bool((buf[:, F:] == 7.0).all())
    assert not ops.gemm_rows8_gated_usable(torch.zeros(2, 2048, dtype=torch.bfloat16, device="cuda"), torch.zeros(64, 2048, dtype=torch.bfloat16, device="cuda"))


@pytest.mark.parametrize("M,N,K,splits", [(96, 1024, 2048, 16), (128, 4096, 1024, 4), (300, 1000, 1032, 3), (512, 1024, 3072, 4),
                                          (70, 130, 520, 3), (1024, 1024, 2048, 2), (257, 72, 136, 2)])
def test_gemm_tc_cut_along_k(ops, M, N, K, splits):
    """The tiled product cut along K: the float32 slices add up to the product (float64 reference of the same
    bfloat16 operands), rows and columns beyond the matrix are not written, tails in M, N and K, and a last
    slice shorter than the others."""
    torch.manual_seed(60 + M)
    a = torch.randn(M, K).to(torch.bfloat16)
    w = (torch.randn(N, K) * 0.5).to(torch.bfloat16)
    a[M - 1, K - 1] = 8.0
    w[N - 1, K - 1] = 8.0
    out = torch.full((splits + 1, M, N), 7.0, dtype=torch.float32, device="cuda")
    ops.gemm_tc_sliced(out[:splits], dev(a), dev(w))
    torch.cuda.synchronize()
    ops.check_tc_errors(out.device)
    ref = a.double() @ w.double().t()
    scale = float(ref.abs().max())
    err = float((out[:splits].double().sum(0).cpu() - ref).abs().max())
    assert err < 2e-5 * scale, (err, scale)
    assert float((out[splits] - 7.0).abs().max()) == 0.0           # the array behind the slices is untouched
    # each slice is the product over its own columns of K
    per = (((K + 63) // 64 + splits - 1) // splits + 1) // 2 * 2 * 64        # slices are whole stages of two steps of 64
    lo = (splits - 1) * per
    last = a[:, lo:].double() @ w[:, lo:].double().t()
    assert float((out[splits - 1].double().cpu() - last).abs().max()) < 2e-5 * scale


def test_gemm_tc_splits_follow_the_tiles(ops):
    """Few tiles: K is cut until about every SM has an item, no slice empty; many tiles: not cut."""
    sms = ops.sm_count(torch.device("cuda"))
    for M, N, K in [(96, 1024, 2048), (128, 4096, 1024), (512, 1024, 3072), (384, 6144, 1024), (2048, 1024, 2048), (65, 1024, 64)]:
        s = ops.gemm_tc_splits(M, N, K)
        tiles = ((M + 127) // 128) * ((N + 127) // 128)
        kb = (K + 63) // 64
        assert 1 <= s <= 16 and tiles * s <= max(sms, tiles)
        if s > 1:
            per = ((kb + s - 1) // s + 1) // 2 * 2
            assert per >= 4 and (s - 1) * per < kb
        if tiles * 4 >= 3 * sms:
            assert s == 1


@pytest.mark.parametrize("mode", [3, 2])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (300, 200, 136), (2048, 1024, 3072), (100, 4096, 1024), (1000, 520, 2048)])
def test_gemm_tc_pairs_of_blocks(ops, M, N, K, mode):
    """Tiles of 256 rows computed by two blocks (`cta_group::2`), forced for every shape: rows that
    leave the second block idle, tails in N that cut its half of W, several tiles per pair."""
    torch.manual_seed(140 + M)
    a = torch.randn(M, K).to(torch.bfloat16)
    w = (torch.randn(N, K) * 0.5).to(torch.bfloat16)
    a[M - 1, K - 1] = 8.0
    w[N - 1, K - 1] = 8.0
    out = torch.full((M, N), 7.0, dtype=torch.float32, device="cuda")
    ops.gemm_tc_set_pair_mode(mode)
    try:
        ops.gemm_tc(out, dev(a), dev(w))
        torch.cuda.synchronize()
    finally:
        ops.gemm_tc_set_pair_mode(1)
    ops.check_tc_errors(out.device)
    ref = a.double() @ w.double().t()
    assert float((out.double().cpu() - ref).abs().max()) < 2e-5 * float(ref.abs().max())


@pytest.mark.parametrize("mode", [3, 2])
def test_gemm_tc_pairs_of_blocks_gated(ops, mode):
    from llmgen_b200.parts.mlp import interleave_gate_up
    torch.manual_seed(141)
    M, F, K = 600, 1040, 1024
    a = torch.randn(M, K).to(torch.bfloat16)
    wg = (torch.randn(F, K) * 0.1).to(torch.bfloat16)
    wu = (torch.randn(F, K) * 0.1).to(torch.bfloat16)
    out = torch.empty(M, F, dtype=torch.bfloat16, device="cuda")
    ops.gemm_tc_set_pair_mode(mode)
    try:
        ops.gemm_tc(out, dev(a), dev(interleave_gate_up(wg, wu)), gated=True)
        torch.cuda.synchronize()
    finally:
        ops.gemm_tc_set_pair_mode(1)
    ops.check_tc_errors(out.device)
    g = a.double() @ wg.double().t()
    u = a.double() @ wu.double().t()
    ref = g / (1 + torch.exp(-g)) * u
    assert float((out.double().cpu() - ref).abs().max()) < 8e-3 * max(1.0, float(ref.abs().max()))


def test_gemm_tc_strided_operands_and_untouched_neighbours(ops):
    torch.manual_seed(60)
    M, N, K = 70, 96, 200
    a_big = torch.randn(M, K + 16).to(torch.bfloat16).cuda()
    w_big = torch.randn(N, K + 8).to(torch.bfloat16).cuda()
    a, w = a_big[:, 8:8 + K], w_big[:, :K]
    big = torch.zeros(M + 2, N + 16, dtype=torch.bfloat16, device="cuda")
    view = big[1:M + 1, 8:8 + N]
    assert ops.gemm_tc_usable(a, w)
    ops.gemm_tc(view, a, w)
    ref = a.double().cpu() @ w.double().cpu().t()
    assert float((view.double().cpu() - ref).abs().max()) < 6e-3 * float(ref.abs().max())
    assert float(big[0].abs().sum()) == 0 and float(big[M + 1].abs().sum()) == 0
    assert float(big[:, :8].abs().sum()) == 0 and float(big[:, 8 + N:].abs().sum()) == 0
    # rows that do not start on 16-byte boundaries are refused, not mis-computed
    assert not ops.gemm_tc_usable(a_big[:, 1:1 + K], w)
    with pytest.raises(ops.KernelError, match="usable"):
        ops.gemm_tc(view, a_big[:, 1:1 + K], w)


@pytest.mark.parametrize("M,F,K", [(3, 48, 64), (130, 176, 80), (2048, 3072, 1024)])
def test_gemm_tc_gated(ops, M, F, K):
    """Gate and up rows interleaved in groups of 16: the epilogue returns silu(gate) * up."""
    from llmgen_b200.parts.mlp import interleave_gate_up
    torch.manual_seed(70)
    a = torch.randn(M, K).to(torch.bfloat16)
    wg = (torch.randn(F, K) * 0.1).to(torch.bfloat16)
    wu = (torch.randn(F, K) * 0.1).to(torch.bfloat16)
    packed = interleave_gate_up(wg, wu)
    out = torch.empty(M, F, dtype=torch.bfloat16, device="cuda")
    ops.gemm_tc(out, dev(a), dev(packed), gated=True)
    g = a.double() @ wg.double().t()
    u = a.double() @ wu.double().t()
    ref = g / (1 + torch.exp(-g)) * u
    assert float((out.double().cpu() - ref).abs().max()) < 8e-3 * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (8, 1024, 2048), (5, 72, 136), (16, 4096, 1024), (17, 200, 1032),
                                   (64, 1024, 3072), (100, 384, 512), (256, 130, 2048), (8, 151936 // 8, 1024)])
@pytest.mark.parametrize("out_dtype", DTYPES)
def test_gemm_skinny_direct(ops, M, N, K, out_dtype):
    """The few-rows tcgen05 product written directly: every padded row count, tails in N and K."""
    torch.manual_seed(150 + M)
    a = torch.randn(M, K).to(torch.bfloat16)
    w = (torch.randn(N, K) * 0.5).to(torch.bfloat16)
    a[M - 1, K - 1] = 8.0
    w[N - 1, K - 1] = 8.0
    out = torch.full((M, N), 7.0, dtype=out_dtype, device="cuda")
    ops.gemm_skinny(out, dev(a), dev(w))
    torch.cuda.synchronize()
    ops.check_tc_errors(out.device)
    ref = a.double() @ w.double().t()
    scale = float(ref.abs().max())
    err = float((out.double().cpu() - ref).abs().max())
    assert err < (2e-5 if out_dtype == torch.float32 else 6e-3) * scale, (err, scale)


@pytest.mark.parametrize("M,N,K,splits", [(8, 1024, 2048, 16), (1, 136, 200, 2), (33, 1024, 3072, 12), (8, 4096, 1024, 4),
                                          (200, 256, 1024, 2), (4, 64, 64, 1)])
def test_gemm_skinny_partial_sums(ops, M, N, K, splits):
    """Cut along K: the slices add up to the product, and the plan never leaves a slice empty."""
    torch.manual_seed(160 + M)
    a = torch.randn(M, K).to(torch.bfloat16)
    w = (torch.randn(N, K) * 0.5).to(torch.bfloat16)
    part = torch.full((splits, M, N), 7.0, dtype=torch.float32, device="cuda")
    ops.gemm_skinny(part, dev(a), dev(w), ops.SKINNY_PARTIAL)
    torch.cuda.synchronize()
    ops.check_tc_errors(part.device)
    ref = a.double() @ w.double().t()
    got = ops.Partials(part).sum().double().cpu()
    assert float((got - ref).abs().max()) < 2e-5 * float(ref.abs().max())
    planned = ops.gemm_skinny_splits(M, N, K)
    kb = (K + 63) // 64
    per = (kb + planned - 1) // planned
    assert planned >= 1 and (planned - 1) * per < kb and planned * M * N * 4 <= max(2 * N * K, M * N * 4)
    with pytest.raises(ops.KernelError, match="empty|slices"):
        ops.gemm_skinny(torch.empty(kb + 1, M, N, dtype=torch.float32, device="cuda"), dev(a), dev(w), ops.SKINNY_PARTIAL)


@pytest.mark.parametrize("M,F,K", [(3, 48, 64), (8, 3072, 1024), (130, 176, 80)])
def test_gemm_skinny_gated(ops, M, F, K):
    from llmgen_b200.parts.mlp import interleave_gate_up
    torch.manual_seed(170)
    a = torch.randn(M, K).to(torch.bfloat16)
    wg = (torch.randn(F, K) * 0.1).to(torch.bfloat16)
    wu = (torch.randn(F, K) * 0.1).to(torch.bfloat16)
    out = torch.empty(M, F, dtype=torch.bfloat16, device="cuda")
    ops.gemm_skinny(out, dev(a), dev(interleave_gate_up(wg, wu)), ops.SKINNY_GATED)
    torch.cuda.synchronize()
    ops.check_tc_errors(out.device)
    g = a.double() @ wg.double().t()
    u = a.double() @ wu.double().t()
    ref = g / (1 + torch.exp(-g)) * u
    assert float((out.double().cpu() - ref).abs().max()) < 8e-3 * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("M,F,K,splits", [(8, 3072, 1024, 4), (1, 48, 128, 2), (33, 176, 256, 4), (64, 1024, 512, 2)])
def test_gemm_skinny_gated_after_the_sum_in_a_cluster(ops, M, F, K, splits):
    from llmgen_b200.parts.mlp import interleave_gate_up
    torch.manual_seed(171 + M)
    a = torch.randn(M, K).to(torch.bfloat16)
    wg = (torch.randn(F, K) * 0.1).to(torch.bfloat16)
    wu = (torch.randn(F, K) * 0.1).to(torch.bfloat16)
    out = torch.full((M, F), 7.0, dtype=torch.bfloat16, device="cuda")
    for _ in range(2):
        ops.gemm_skinny(out, dev(a), dev(interleave_gate_up(wg, wu)), ops.SKINNY_CLUSTER_GATED, splits=splits)
    torch.cuda.synchronize()
    ops.check_tc_errors(out.device)
    g = a.double() @ wg.double().t()
    u = a.double() @ wu.double().t()
    ref = g / (1 + torch.exp(-g)) * u
    assert float((out.double().cpu() - ref).abs().max()) < 8e-3 * max(1.0, float(ref.abs().max()))
    with pytest.raises(ops.KernelError, match="2 or 4|slices"):
        ops.gemm_skinny(out, dev(a), dev(interleave_gate_up(wg, wu)), ops.SKINNY_CLUSTER_GATED, splits=8)


def test_gemm_skinny_refuses_what_it_cannot_do(ops):
    w = torch.zeros(64, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ops.KernelError, match="above 256"):
        ops.gemm_skinny(torch.empty(257, 64, dtype=torch.bfloat16, device="cuda"),
                        torch.zeros(257, 64, dtype=torch.bfloat16, device="cuda"), w)
    big = torch.zeros(4, 80, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ops.KernelError, match="usable"):
        ops.gemm_skinny(torch.empty(4, 64, dtype=torch.bfloat16, device="cuda"), big[:, 1:65], w)


@pytest.mark.parametrize("dtype", DTYPES)
def test_consumers_add_up_partial_sums(ops, dtype):
    """add_rmsnorm, silu_mul and attn_prep given float32 slices equal the same kernels given the sum."""
    torch.manual_seed(180)
    n, H, S = 5, 136, 3
    slices = torch.randn(S, n, H).cuda()
    total = slices.sum(0)
    resid = torch.randn(n, H).cuda()
    w = (1 + 0.1 * torch.randn(H)).cuda()
    r1, r2 = resid.clone(), resid.clone()
    o1 = torch.empty(n, H, dtype=dtype, device="cuda")
    o2 = torch.empty_like(o1)
    ops.add_rmsnorm(r1, ops.Partials(slices), w, o1, 1e-5)
    r2 += total
    ops.add_rmsnorm(r2, None, w, o2, 1e-5)
    assert torch.allclose(r1, r2, atol=1e-5) and torch.allclose(o1.float(), o2.float(), atol=tol(dtype))
    rows = torch.tensor([4, 0, 2], dtype=torch.int32, device="cuda")
    g1 = torch.empty(3, H, dtype=dtype, device="cuda")
    ops.add_rmsnorm(resid.clone(), ops.Partials(slices), w, g1, 1e-5, rows=rows)
    assert torch.allclose(g1.float(), o2[rows.long()].float(), atol=tol(dtype))
    # gated activation, groups of 16
    F = 48
    gu = torch.randn(S, n, 2 * F).cuda()
    a1 = torch.empty(n, F, dtype=dtype, device="cuda")
    a2 = torch.empty_like(a1)
    ops.silu_mul(a1, ops.Partials(gu), group=16)
    ops.silu_mul(a2, gu.sum(0).to(dtype).contiguous(), group=16)
    assert torch.allclose(a1.float(), a2.float(), atol=tol(dtype, 4))
    # q/k norm + rotary + cache write
    nq, nkv, hd, page = 4, 2, 32, 8
    width = (nq + 2 * nkv) * hd
    qkv = torch.randn(S, n, width).cuda()
    whole = qkv.sum(0).to(dtype).contiguous()
    pos = torch.arange(n, dtype=torch.int32, device="cuda") + 3
    slots = torch.tensor([9, 2, -1, 17, 4], dtype=torch.int32, device="cuda")
    cos, sin = plain.rope_tables(64, hd, 10000.0)
    cos, sin = dev(cos.float()), dev(sin.float())
    qg, kg = (1 + 0.1 * torch.randn(hd)).cuda(), (1 + 0.1 * torch.randn(hd)).cuda()
    caches = [[torch.zeros(4, nkv, page, hd, dtype=dtype, device="cuda") for _ in range(2)] for _ in range(2)]
    q1 = torch.empty(n, nq * hd, dtype=dtype, device="cuda")
    ops.attn_prep(ops.Partials(qkv), caches[0][0], caches[0][1], pos, slots, cos, sin, qg, kg, nq, nkv, hd, hd, page, 1e-6, q_out=q1)
    ops.attn_prep(whole, caches[1][0], caches[1][1], pos, slots, cos, sin, qg, kg, nq, nkv, hd, hd, page, 1e-6)
    assert torch.allclose(q1.float(), whole[:, : nq * hd].float(), atol=tol(dtype, 4))
    for a, b in zip(caches[0], caches[1]):
        assert torch.allclose(a.float(), b.float(), atol=tol(dtype, 4))



@pytest.mark.parametrize("M", [1, 2, 3, 4])
@pytest.mark.parametrize("out_dtype", DTYPES)
def test_gemv_bf16(ops, M, out_dtype):
    torch.manual_seed(7)
    N, K = 131, 520
    a = torch.randn(M, K).to(torch.bfloat16)
    w = (torch.randn(N, K) * 0.1).to(torch.bfloat16)
    out = torch.empty(M, N, dtype=out_dtype, device="cuda")
    assert ops.gemv_usable(dev(a), dev(w))
    ops.gemv_bf16(out, dev(a), dev(w))
    ref = a.double() @ w.double().t()
    assert float((out.double().cpu() - ref).abs().max()) < (1e-4 if out_dtype == torch.float32 else 3e-2)
    assert not ops.gemv_usable(dev(torch.zeros(5, K, dtype=torch.bfloat16)), dev(w))
    assert not ops.gemv_usable(dev(torch.zeros(2, 12, dtype=torch.bfloat16)), dev(torch.zeros(4, 12, dtype=torch.bfloat16)))
    with pytest.raises(ops.KernelError, match="multiple of 8"):
        ops.gemv_bf16(torch.empty(1, 4, dtype=out_dtype, device="cuda"), dev(torch.zeros(1, 12, dtype=torch.bfloat16)),
                      dev(torch.zeros(4, 12, dtype=torch.bfloat16)))


# ------------------------------------------------------------------ attention
def paged_case(seqs, nq, nkv, hd, page, dtype, seed, sharpen=None):
    """seqs: [(ctx, q_len)].  Builds a shuffled paged cache and q; returns tensors and the plain result."""
    g = torch.Generator().manual_seed(seed)
    max_blocks = max((c + page - 1) // page for c, _ in seqs) + 1
    n_pages = sum((c + page - 1) // page for c, _ in seqs) + 3
    order = list(range(n_pages))
    random.Random(seed).shuffle(order)
    kc = torch.randn(n_pages, nkv, page, hd, generator=g).to(dtype)      # unused slots hold noise
    vc = torch.randn(n_pages, nkv, page, hd, generator=g).to(dtype)
    bt = torch.zeros(len(seqs), max_blocks, dtype=torch.int32)
    T = sum(q for _, q in seqs)
    q = torch.randn(T, nq, hd, generator=g).to(dtype)
    ref = torch.zeros(T, nq, hd)
    cu, ctxs, t = [0], [], 0
    for s, (ctx, q_len) in enumerate(seqs):
        nb = (ctx + page - 1) // page
        pages = [order.pop() for _ in range(nb)]
        bt[s, :nb] = torch.tensor(pages, dtype=torch.int32)
        ctxs.append(ctx)
        if ctx >= q_len and ctx > 0:
            k_seq = torch.stack([kc[pages[p // page], :, p % page] for p in range(ctx)]).float()
            v_seq = torch.stack([vc[pages[p // page], :, p % page] for p in range(ctx)]).float()
            if sharpen is not None:
                sharpen(s, ctx, q_len, q, t, k_seq, kc, pages, page)
            q_full = torch.zeros(ctx, nq, hd)
            q_full[ctx - q_len:] = q[t:t + q_len].float()
            ref[t:t + q_len] = plain.causal_attention(q_full, k_seq, v_seq, 1.0 / math.sqrt(hd), sharpen.window if sharpen is not None and hasattr(sharpen, "window") else None)[ctx - q_len:]
        t += q_len
        cu.append(t)
    return q, kc, vc, bt, torch.tensor(ctxs, dtype=torch.int32), torch.tensor(cu, dtype=torch.int32), ref, max_blocks


def run_attention(ops, q, kc, vc, bt, ctxs, cu, max_blocks, nq, nkv, hd, page, window=0, parts=1, part_size=0):
    T = q.shape[0]
    bq = ops.attention_tile_queries(nq, nkv)
    seq, q0 = [], []
    for s in range(len(ctxs)):
        n = int(cu[s + 1] - cu[s])
        for start in range(0, max(n, 1), bq):
            seq.append(s)
            q0.append(start)
    out = torch.full((T, nq * hd), 9.0, dtype=q.dtype, device="cuda")
    scratch = None
    if parts > 1:
        scratch = torch.empty(ops.attention_scratch_floats(T, nq, hd, parts), dtype=torch.float32, device="cuda")
    qd = dev(q.view(T, nq * hd))
    ops.paged_attention(out, qd, nq * hd, dev(kc), dev(vc), dev(bt), max_blocks, dev(ctxs), dev(cu),
                        dev(torch.tensor(seq, dtype=torch.int32)), dev(torch.tensor(q0, dtype=torch.int32)), len(seq), T,
                        nq, nkv, hd, page, window, 1.0 / math.sqrt(hd), parts, part_size, scratch)
    return out.float().cpu().view(T, nq, hd)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,hd,page", [(4, 2, 64, 16), (8, 1, 32, 32), (6, 2, 48, 16), (16, 8, 128, 16),
                                            (3, 3, 16, 8), (40, 2, 16, 16), (2, 2, 256, 64)])
def test_paged_attention_mixed_batch(ops, dtype, nq, nkv, hd, page):
    # the reference's own mixed case (src/backend/cpu/attention.zig:188-251): the tail of a
    # prompt (ctx 70, 30 queries), a decoded token (ctx 41), a padding row (ctx 0); plus a whole
    # prompt that ends on a page's edge and a single first token
    seqs = [(70, 30), (41, 1), (0, 1), (4 * page, 4 * page), (1, 1), (150, 100)]
    q, kc, vc, bt, ctxs, cu, ref, mb = paged_case(seqs, nq, nkv, hd, page, dtype, 11)
    got = run_attention(ops, q, kc, vc, bt, ctxs, cu, mb, nq, nkv, hd, page)
    assert float((got - ref).abs().max()) < tol(dtype, 3)
    assert float(got[31].abs().max()) == 0.0        # the padding row gives zeros


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("parts,part_size", [(1, 0), (6, 64), (3, 128), (5, 0), (16, 0), (2, 512)])
def test_flash_decoding_split(ops, dtype, parts, part_size):
    # a fixed part_size must cover the longest context (parts * part_size >= 333); 0 splits evenly
    nq, nkv, hd, page = 4, 2, 128, 16
    seqs = [(150, 1), (1, 1), (0, 1), (333, 1), (64, 1), (65, 1)]
    q, kc, vc, bt, ctxs, cu, ref, mb = paged_case(seqs, nq, nkv, hd, page, dtype, 12)
    got = run_attention(ops, q, kc, vc, bt, ctxs, cu, mb, nq, nkv, hd, page, parts=parts, part_size=part_size)
    assert float((got - ref).abs().max()) < tol(dtype, 3)
    assert float(got[2].abs().max()) == 0.0


class FarKey:
    """Scales one key (and the queries) so that a single far score stands out: if that key is
    missed (a page's edge, a part's boundary, the first key) the output is visibly wrong."""
    def __init__(self, where):
        self.where = where

    def __call__(self, s, ctx, q_len, q, t, k_seq, kc, pages, page):
        j = self.where(ctx)
        if not 0 <= j < ctx:
            return
        direction = q[t + q_len - 1, 0].float()
        boost = (6.0 * direction / direction.norm()).to(kc.dtype)
        kc[pages[j // page], :, j % page] = boost
        k_seq[j] = boost.float()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("where", [lambda c: 0, lambda c: 15, lambda c: 16, lambda c: c - 1, lambda c: 255, lambda c: 256,
                                   lambda c: c // 2])
def test_far_key_among_hundreds(ops, dtype, where):
    nq, nkv, hd, page = 2, 1, 64, 16
    seqs = [(700, 1), (513, 3)]
    q, kc, vc, bt, ctxs, cu, ref, mb = paged_case(seqs, nq, nkv, hd, page, dtype, 13, sharpen=FarKey(where))
    for parts, part_size in ((1, 0), (4, 0), (3, 256)):
        if parts > 1:       # split runs are for single-token rows
            seqs1 = [(700, 1)]
            q1, kc1, vc1, bt1, ctxs1, cu1, ref1, mb1 = paged_case(seqs1, nq, nkv, hd, page, dtype, 13, sharpen=FarKey(where))
            got = run_attention(ops, q1, kc1, vc1, bt1, ctxs1, cu1, mb1, nq, nkv, hd, page, parts=parts, part_size=part_size)
            assert float((got - ref1).abs().max()) < tol(dtype, 3)
        else:
            got = run_attention(ops, q, kc, vc, bt, ctxs, cu, mb, nq, nkv, hd, page)
            assert float((got - ref).abs().max()) < tol(dtype, 3)


class WindowEdge(FarKey):
    def __init__(self, window, offset):
        super().__init__(lambda ctx: ctx - 1 - window + offset)   # offset 0: just outside; 1: just inside
        self.window = window


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 7, 16, 40, 100])
@pytest.mark.parametrize("offset", [0, 1])
def test_window_edge(ops, dtype, window, offset):
    """The key one place outside the window must not be seen, the one just inside must."""
    nq, nkv, hd, page = 6, 2, 48, 16
    seqs = [(130, 1), (97, 33), (40, 40), (0, 1)]
    q, kc, vc, bt, ctxs, cu, ref, mb = paged_case(seqs, nq, nkv, hd, page, dtype, 14, sharpen=WindowEdge(window, offset))
    got = run_attention(ops, q, kc, vc, bt, ctxs, cu, mb, nq, nkv, hd, page, window=window)
    assert float((got - ref).abs().max()) < tol(dtype, 3)


# ------------------------------------------------- tensor-core attention (prompts, bfloat16)
def run_attention_tc(ops, q, kc, vc, bt, ctxs, cu, max_blocks, nq, nkv, hd, page, window=0, v_lbo=0, v_sbo=0):
    T = q.shape[0]
    bq = ops.attention_tc_tile_queries(nq, nkv, hd, page)
    assert bq > 0
    seq, q0 = [], []
    for s in range(len(ctxs)):
        n = int(cu[s + 1] - cu[s])
        for start in range(0, max(n, 1), bq):
            seq.append(s)
            q0.append(start)
    out = torch.full((T, nq * hd), 9.0, dtype=q.dtype, device="cuda")
    qd = dev(q.view(T, nq * hd))
    ops.attention_tc(out, qd, nq * hd, dev(kc), dev(vc), dev(bt), max_blocks, dev(ctxs), dev(cu),
                     dev(torch.tensor(seq, dtype=torch.int32)), dev(torch.tensor(q0, dtype=torch.int32)), len(seq), T,
                     nq, nkv, hd, page, window, 1.0 / math.sqrt(hd), v_lbo, v_sbo)
    torch.cuda.synchronize()
    ops.check_tc_errors(out.device)
    return out.float().cpu().view(T, nq, hd)


TC_SHAPES = [(4, 2, 64, 16), (16, 8, 128, 16), (8, 1, 128, 32), (6, 2, 64, 16), (2, 2, 128, 64), (12, 2, 128, 128)]


@pytest.mark.parametrize("nq,nkv,hd,page", TC_SHAPES)
def test_attention_tc_mixed_batch(ops, nq, nkv, hd, page):
    """Whole prompts over several key tiles, prompt tails, single tokens, a padding row, a prompt that
    ends on a tile's edge; groups of 1, 2, 3, 6 and 8 heads."""
    dtype = torch.bfloat16
    seqs = [(70, 30), (41, 1), (0, 1), (256, 256), (1, 1), (150, 100), (700, 390), (129, 129)]
    q, kc, vc, bt, ctxs, cu, ref, mb = paged_case(seqs, nq, nkv, hd, page, dtype, 21)
    got = run_attention_tc(ops, q, kc, vc, bt, ctxs, cu, mb, nq, nkv, hd, page)
    assert float((got - ref).abs().max()) < tol(dtype, 3)
    assert float(got[31].abs().max()) == 0.0        # the padding row gives zeros


def test_attention_tc_long_prompt(ops):
    """One prompt of 2,048 tokens at the heads of the benchmark's shape: 16 key tiles, 32 query tiles."""
    nq, nkv, hd, page = 16, 8, 128, 16
    seqs = [(2048, 2048)]
    q, kc, vc, bt, ctxs, cu, ref, mb = paged_case(seqs, nq, nkv, hd, page, torch.bfloat16, 22)
    got = run_attention_tc(ops, q, kc, vc, bt, ctxs, cu, mb, nq, nkv, hd, page)
    assert float((got - ref).abs().max()) < tol(torch.bfloat16, 3)


@pytest.mark.parametrize("where", [lambda c: 0, lambda c: 15, lambda c: 16, lambda c: 127, lambda c: 128, lambda c: c - 1,
                                   lambda c: 255, lambda c: 256, lambda c: c // 2])
def test_attention_tc_far_key(ops, where):
    nq, nkv, hd, page = 2, 1, 64, 16
    seqs = [(700, 1), (513, 3), (640, 200)]
    q, kc, vc, bt, ctxs, cu, ref, mb = paged_case(seqs, nq, nkv, hd, page, torch.bfloat16, 23, sharpen=FarKey(where))
    got = run_attention_tc(ops, q, kc, vc, bt, ctxs, cu, mb, nq, nkv, hd, page)
    assert float((got - ref).abs().max()) < tol(torch.bfloat16, 3)


class RisingKeys:
    """Keys along the last query's direction with a length that grows with the position: the row maximum
    rises from tile to tile, slowly (the reference maximum of the tensor-core kernel lags behind it) or
    fast (it moves on every tile), and the last keys carry nearly all the weight."""
    def __init__(self, top):
        self.top = top

    def __call__(self, s, ctx, q_len, q, t, k_seq, kc, pages, page):
        direction = q[t + q_len - 1, 0].float()
        unit = direction / direction.norm()
        for j in range(ctx):
            key = (unit * (self.top * (j + 1) / ctx)).to(kc.dtype)
            kc[pages[j // page], :, j % page] = key
            k_seq[j] = key.float()


@pytest.mark.parametrize("top", [6.0, 14.0, 30.0, 70.0])
def test_attention_tc_rising_scores(ops, top):
    nq, nkv, hd, page = 4, 2, 64, 16
    seqs = [(700, 1), (1030, 300), (640, 640)]
    q, kc, vc, bt, ctxs, cu, ref, mb = paged_case(seqs, nq, nkv, hd, page, torch.bfloat16, 25, sharpen=RisingKeys(top))
    got = run_attention_tc(ops, q, kc, vc, bt, ctxs, cu, mb, nq, nkv, hd, page)
    assert float((got - ref).abs().max()) < tol(torch.bfloat16, 3)


@pytest.mark.parametrize("window", [1, 7, 16, 40, 100, 200])
@pytest.mark.parametrize("offset", [0, 1])
def test_attention_tc_window_edge(ops, window, offset):
    nq, nkv, hd, page = 6, 2, 64, 16
    seqs = [(130, 1), (97, 33), (40, 40), (0, 1), (400, 250)]
    q, kc, vc, bt, ctxs, cu, ref, mb = paged_case(seqs, nq, nkv, hd, page, torch.bfloat16, 24, sharpen=WindowEdge(window, offset))
    got = run_attention_tc(ops, q, kc, vc, bt, ctxs, cu, mb, nq, nkv, hd, page, window=window)
    assert float((got - ref).abs().max()) < tol(torch.bfloat16, 3)


def test_attention_tc_refuses_what_it_cannot_do(ops):
    assert ops.attention_tc_tile_queries(4, 2, 48, 16) == 0       # head_dim
    assert ops.attention_tc_tile_queries(4, 2, 64, 8) == 0        # page size
    assert ops.attention_tc_tile_queries(4, 3, 64, 16) == 0       # heads
    z = torch.zeros(1, 96, dtype=torch.bfloat16, device="cuda")
    zi = torch.zeros(4, dtype=torch.int32, device="cuda")
    with pytest.raises(ops.KernelError, match="not taken"):
        ops.attention_tc(z, z, 96, z.view(1, 1, 2, 48), z.view(1, 1, 2, 48), zi, 1, zi, zi, zi, zi, 1, 1, 2, 1, 48, 2, 0, 1.0)


# ------------------------------------------------- decode attention (single tokens, bfloat16)
def run_attention_decode(ops, q, kc, vc, bt, ctxs, cu, max_blocks, nq, nkv, hd, page, window=0, parts=1, counters=None,
                         bound=None):
    S = len(ctxs)
    T = q.shape[0]
    assert T == S
    out = torch.full((T, nq * hd), 9.0, dtype=q.dtype, device="cuda")
    scratch = None
    if parts > 1:
        scratch = torch.empty(ops.attention_decode_scratch_floats(S, nq, hd, parts), dtype=torch.float32, device="cuda")
        if counters is None:
            counters = torch.zeros(ops.attention_decode_counters(S, nq, nkv), dtype=torch.int32, device="cuda")
    qd = dev(q.view(T, nq * hd))
    ops.attention_decode(out, qd, nq * hd, dev(kc), dev(vc), dev(bt), max_blocks, dev(ctxs), dev(cu), S, nq, nkv, hd,
                         page, window, 1.0 / math.sqrt(hd), parts, int(max(ctxs)) if bound is None else bound, scratch, counters)
    return out.float().cpu().view(T, nq, hd)


@pytest.mark.parametrize("nq,nkv,hd,page", [(4, 2, 128, 16), (16, 8, 128, 16), (8, 1, 64, 32), (6, 2, 64, 16), (3, 3, 128, 8),
                                            (40, 2, 64, 16), (24, 2, 128, 16), (64, 8, 128, 16), (8, 2, 128, 32)])
@pytest.mark.parametrize("parts", [1, 4, 7, 37])
def test_attention_decode(ops, nq, nkv, hd, page, parts):
    """Single tokens against contexts of 1 to 700 keys and a padding row, one part and many (more
    parts than some contexts have keys); groups of 1, 2, 3, 8, 12 and 20 heads; the counters are
    left zero, so a second launch with the same counters gives the same result."""
    dtype = torch.bfloat16
    seqs = [(150, 1), (1, 1), (0, 1), (333, 1), (64, 1), (65, 1), (700, 1), (9, 1)]
    q, kc, vc, bt, ctxs, cu, ref, mb = paged_case(seqs, nq, nkv, hd, page, dtype, 31)
    counters = torch.zeros(ops.attention_decode_counters(len(seqs), nq, nkv), dtype=torch.int32, device="cuda")
    # up to 8 parts merge through the shared memory of a cluster, more through global memory and a ticket;
    # the second round forces the ticket for every number of parts
    for through_cluster in (True, False):
        ops.attention_decode_set_cluster_merge(through_cluster)
        try:
            got = run_attention_decode(ops, q, kc, vc, bt, ctxs, cu, mb, nq, nkv, hd, page, parts=parts, counters=counters)
        finally:
            ops.attention_decode_set_cluster_merge(True)
        assert float((got - ref).abs().max()) < tol(dtype, 3)
        assert float(got[2].abs().max()) == 0.0
        assert int(counters.abs().sum()) == 0


@pytest.mark.parametrize("parts", [1, 3, 12])
def test_attention_decode_reports_a_sequence_beyond_its_bound(ops, parts):
    """A launch sized for at most 64 keys meets a sequence of 700: the kernel touches nothing for it (its page
    ids would not fit the shared array), raises the device flag, leaves the counters zero, and the other
    sequences of the launch are still right."""
    nq, nkv, hd, page = 4, 2, 128, 16
    seqs = [(40, 1), (700, 1), (64, 1)]
    q, kc, vc, bt, ctxs, cu, ref, mb = paged_case(seqs, nq, nkv, hd, page, torch.bfloat16, 33)
    counters = torch.zeros(ops.attention_decode_counters(len(seqs), nq, nkv), dtype=torch.int32, device="cuda")
    for through_cluster in (True, False):
        ops.attention_decode_set_cluster_merge(through_cluster)
        try:
            got = run_attention_decode(ops, q, kc, vc, bt, ctxs, cu, mb, nq, nkv, hd, page, parts=parts, counters=counters, bound=64)
        finally:
            ops.attention_decode_set_cluster_merge(True)
        with pytest.raises(ops.KernelError, match="longer than the bound"):
            ops.check_tc_errors(torch.device("cuda:0"))
        ops.check_tc_errors(torch.device("cuda:0"))                  # the flag was cleared
        assert int(counters.abs().sum()) == 0
        for s in (0, 2):
            assert float((got[s] - ref[s]).abs().max()) < tol(torch.bfloat16, 3)


def test_attention_decode_batch_64(ops):
    """64 sequences of 577 to 640 keys at the benchmark's head geometry (168 MB of cache would be the
    full model's 28 layers; this is one layer, 5.9 MB per kv head pair): one part and two."""
    nq, nkv, hd, page = 16, 8, 128, 16
    seqs = [(640 - s, 1) for s in range(64)]
    q, kc, vc, bt, ctxs, cu, ref, mb = paged_case(seqs, nq, nkv, hd, page, torch.bfloat16, 37)
    for parts in (1, 2):
        got = run_attention_decode(ops, q, kc, vc, bt, ctxs, cu, mb, nq, nkv, hd, page, parts=parts)
        assert float((got - ref).abs().max()) < tol(torch.bfloat16, 3)


@pytest.mark.parametrize("nq,nkv,hd,page,rot", [(4, 2, 128, 16, 128), (16, 8, 128, 16, 128), (6, 2, 64, 16, 64), (20, 2, 64, 32, 64),
                                                (4, 2, 128, 16, 64), (2, 1, 64, 8, 0), (64, 8, 128, 16, 128), (8, 2, 128, 16, 128)])
@pytest.mark.parametrize("parts", [1, 5])
@pytest.mark.parametrize("sliced", [False, True])
def test_attention_decode_makes_q_k_v_itself(ops, nq, nkv, hd, page, rot, parts, sliced):
    """Given the packed projection rows, the kernel equals attn_prep followed by itself: same outputs,
    same cache contents (the newest key and value of every sequence land in their slots)."""
    dtype = torch.bfloat16
    seqs = [(150, 1), (1, 1), (0, 1), (333, 1), (64, 1), (65, 1), (17, 1)]
    S = len(seqs)
    _, kc, vc, bt, ctxs, cu, _, mb = paged_case(seqs, nq, nkv, hd, page, dtype, 35)
    g = torch.Generator().manual_seed(36)
    width = (nq + 2 * nkv) * hd
    slices = torch.randn(3, S, width, generator=g) * 0.6
    whole = slices.sum(0).to(dtype)
    positions = torch.tensor([max(c - 1, 0) for c, _ in seqs], dtype=torch.int32)
    slots = torch.tensor([int(bt[s, (c - 1) // page]) * page + (c - 1) % page if c > 0 else -1 for s, (c, _) in enumerate(seqs)],
                         dtype=torch.int32)
    qg, kg = (1 + 0.2 * torch.randn(hd, generator=g)), (1 + 0.2 * torch.randn(hd, generator=g))
    cos = sin = None
    if rot:
        c64, s64 = plain.rope_tables(400, rot, 10000.0)
        cos, sin = dev(c64.float()), dev(s64.float())
    scale = 1.0 / math.sqrt(hd)
    args = dict(positions=dev(positions), slots=dev(slots), cos=cos, sin=sin, q_gain=dev(qg), k_gain=dev(kg), eps=1e-6)
    # the two kernels one after the other
    k1, v1 = dev(kc), dev(vc)
    q1 = torch.empty(S, nq * hd, dtype=dtype, device="cuda")
    ops.attn_prep(dev(whole), k1, v1, args["positions"], args["slots"], cos, sin, args["q_gain"], args["k_gain"],
                  nq, nkv, hd, rot, page, 1e-6, q_out=q1)
    out1 = torch.full((S, nq * hd), 9.0, dtype=dtype, device="cuda")
    scratch = torch.empty(max(1, ops.attention_decode_scratch_floats(S, nq, hd, parts)), dtype=torch.float32, device="cuda")
    counters = torch.zeros(ops.attention_decode_counters(S, nq, nkv), dtype=torch.int32, device="cuda")
    common = (dev(bt), mb, dev(ctxs), dev(cu), S, nq, nkv, hd, page, 0, scale, parts, int(max(ctxs)), scratch, counters)
    ops.attention_decode(out1, q1, nq * hd, k1, v1, *common)
    # the one kernel
    k2, v2 = dev(kc), dev(vc)
    out2 = torch.full((S, nq * hd), 9.0, dtype=dtype, device="cuda")
    packed = ops.Partials(dev(slices)) if sliced else dev(whole)
    ops.attention_decode(out2, None, 0, k2, v2, *common, packed=packed, nk=nkv, rot=rot, **args)
    torch.cuda.synchronize()
    assert float((out1.float() - out2.float()).abs().max()) < tol(dtype, 2)
    assert float((k1.float() - k2.float()).abs().max()) < tol(dtype, 2 if sliced else 0.5)
    assert float((v1.float() - v2.float()).abs().max()) < tol(dtype, 2 if sliced else 0.01)
    assert float(out2[2].abs().max()) == 0.0 and int(counters.abs().sum()) == 0


@pytest.mark.parametrize("where", [lambda c: 0, lambda c: 15, lambda c: 16, lambda c: c - 1, lambda c: 255, lambda c: 256,
                                   lambda c: c // 2])
@pytest.mark.parametrize("parts", [1, 3, 8])
def test_attention_decode_far_key(ops, where, parts):
    nq, nkv, hd, page = 2, 1, 64, 16
    seqs = [(700, 1), (513, 1)]
    q, kc, vc, bt, ctxs, cu, ref, mb = paged_case(seqs, nq, nkv, hd, page, torch.bfloat16, 33, sharpen=FarKey(where))
    got = run_attention_decode(ops, q, kc, vc, bt, ctxs, cu, mb, nq, nkv, hd, page, parts=parts)
    assert float((got - ref).abs().max()) < tol(torch.bfloat16, 3)


@pytest.mark.parametrize("window", [1, 7, 16, 40, 100])
@pytest.mark.parametrize("offset", [0, 1])
@pytest.mark.parametrize("parts", [1, 3])
def test_attention_decode_window_edge(ops, window, offset, parts):
    nq, nkv, hd, page = 6, 2, 64, 16
    seqs = [(130, 1), (97, 1), (40, 1), (0, 1)]
    q, kc, vc, bt, ctxs, cu, ref, mb = paged_case(seqs, nq, nkv, hd, page, torch.bfloat16, 34, sharpen=WindowEdge(window, offset))
    got = run_attention_decode(ops, q, kc, vc, bt, ctxs, cu, mb, nq, nkv, hd, page, window=window, parts=parts)
    assert float((got - ref).abs().max()) < tol(torch.bfloat16, 3)


def test_attention_refuses_what_it_cannot_do(ops):
    z = torch.zeros(1, 20, device="cuda")
    zi = torch.zeros(4, dtype=torch.int32, device="cuda")
    with pytest.raises(ops.KernelError, match="head_dim"):
        ops.paged_attention(z, z, 20, z, z, zi, 1, zi, zi, zi, zi, 1, 1, 1, 1, 20, 16, 0, 1.0)
    with pytest.raises(ops.KernelError, match="multiple"):
        ops.paged_attention(z, z, 48, z, z, zi, 1, zi, zi, zi, zi, 1, 1, 3, 2, 16, 16, 0, 1.0)


# ------------------------------------------------------------------ sampling
@pytest.mark.parametrize("V", [1000, 301, 151936])
def test_sample_greedy_finds_the_peak_in_every_segment(ops, V):
    torch.manual_seed(8)
    peaks = [0, 1, V // 32, V // 2 + 3, V - 2, V - 1]
    logits = torch.randn(len(peaks), V)
    for r, p in enumerate(peaks):
        logits[r, p] = 50.0
    logits[1, 7] = 50.0       # a tie: the smaller id wins
    out = torch.zeros(len(peaks), dtype=torch.int32, device="cuda")
    scratch = ops.sample_scratch(len(peaks), "cuda")
    seed = torch.tensor([1234], dtype=torch.int64, device="cuda")
    ops.sample(out, dev(logits), dev(torch.zeros(len(peaks))), seed, scratch)
    assert out.cpu().tolist() == peaks


def test_sample_temperature_matches_the_plain_sampler(ops):
    torch.manual_seed(9)
    V, S = 301, 6
    logits = torch.randn(S, V) * 2
    temps = torch.tensor([0.7, 0.0, 1.0, 0.3, 2.5, 0.7])
    step_seed = 0x5EED + 0x9E3779B97F4A7C15
    out = torch.zeros(S, dtype=torch.int32, device="cuda")
    scratch = ops.sample_scratch(S, "cuda")
    seed = torch.tensor([step_seed - (1 << 64) if step_seed >= (1 << 63) else step_seed], dtype=torch.int64, device="cuda")
    ops.sample(out, dev(logits), dev(temps), seed, scratch)
    got = out.cpu().tolist()
    for row in range(S):
        if temps[row] <= 0:
            assert got[row] == int(logits[row].argmax())
            continue
        scores = plain.gumbel_scores(logits[row], float(temps[row]), step_seed, row)
        # the chosen id's perturbed score is the largest, up to the rounding of log on the two sides
        assert float(scores.max() - scores[got[row]]) < 1e-4
    out2 = torch.zeros_like(out)
    ops.sample(out2, dev(logits), dev(temps), seed, scratch)
    assert torch.equal(out, out2)                                  # same seed, same draw
    seed2 = torch.tensor([99], dtype=torch.int64, device="cuda")
    draws = []
    flat = torch.zeros(1, V)
    for s in range(300):
        seed2.fill_(s * 7919 + 1)
        one = torch.zeros(1, dtype=torch.int32, device="cuda")
        ops.sample(one, dev(flat), dev(torch.ones(1)), seed2, scratch)
        draws.append(int(one.item()))
    assert len(set(draws)) > 150                                   # uniform logits: draws spread over the vocabulary


@pytest.mark.parametrize("V", [1000, 301, 151936])
def test_sample_ids_equal_the_plain_sampler(ops, V):
    """Greedy and temperature rows, in rows that start on 16-byte boundaries and in rows that do not (a row
    stride that is no multiple of 4): the id is the plain sampler's whenever its two best scores are apart by
    more than the rounding of log."""
    torch.manual_seed(12 + V)
    S = 3
    temps = torch.tensor([0.6, 0.0, 1.7])
    step_seed = (0xC0FFEE * 7919 + V) & ((1 << 63) - 1)
    for pad in (0, 3):
        wide = (torch.randn(S, V + pad) * 2).cuda()
        logits = wide[:, :V]
        out = torch.full((S,), -1, dtype=torch.int32, device="cuda")
        seed = torch.tensor([step_seed], dtype=torch.int64, device="cuda")
        ops.sample(out, logits, dev(temps), seed, ops.sample_scratch(S, "cuda"))
        got = out.cpu().tolist()
        for row in range(S):
            x = logits[row].cpu()
            if temps[row] <= 0:
                assert got[row] == int(x.argmax())
                continue
            scores = plain.gumbel_scores(x, float(temps[row]), step_seed, row)
            top = scores.topk(2)
            if float(top.values[0] - top.values[1]) > 1e-5:
                assert got[row] == int(top.indices[0])
            else:
                assert got[row] in top.indices.tolist()


def test_sample_of_rows_without_a_comparable_score(ops):
    """A row of NaN (a fault upstream) gives id 0, not an id outside the vocabulary; a row whose only finite
    score is its last one finds it; -inf everywhere is a tie that the smallest id wins."""
    V = 777
    logits = torch.full((3, V), float("nan"))
    logits[1, :] = float("-inf")
    logits[1, V - 1] = -3.0
    logits[2, :] = float("-inf")
    for temp in (0.0, 0.9):
        out = torch.full((3,), -1, dtype=torch.int32, device="cuda")
        seed = torch.tensor([5], dtype=torch.int64, device="cuda")
        ops.sample(out, dev(logits), dev(torch.full((3,), temp)), seed, ops.sample_scratch(3, "cuda"))
        assert out.cpu().tolist() == [0, V - 1, 0]

