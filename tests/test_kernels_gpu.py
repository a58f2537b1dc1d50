"""Each kernel alone against a plain float32/float64 restatement of the same operation,
at sizes other than the engine tests' (odd widths, head sizes in steps of 16, groups of
1..7, vocabularies that are no power of two)."""
import numpy as np
import pytest
import torch

import plain_qwen2 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ops():
    from coheryn_ai_studio_b200 import ops as o
    return o


def t32(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


@pytest.mark.parametrize("table_dtype", [torch.float32, torch.bfloat16])
def test_embed_gather(table_dtype):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(301, 72, generator=g).to(table_dtype).to(DEV)
    ids = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 72, dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops().embed_gather(table, ids, out, status)
    assert torch.equal(out, table.float()[ids.long()]) and status.item() == 0
    bad = torch.tensor([3, 301], dtype=torch.int32, device=DEV)
    ops().embed_gather(table, bad, out[:2], status)
    assert status.item() == 1


@pytest.mark.parametrize("H", [72, 1536, 3000, 1537])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("splits", [1, 3, 12])
def test_add_rmsnorm_takes_partial_sums(H, dtype, splits):
    """The delta as a float32 stack of partial sums: added in order, then to the residual."""
    rng = np.random.default_rng(H + splits)
    resid = rng.standard_normal((5, H)).astype(np.float32) * 3
    parts = rng.standard_normal((splits, 5, H)).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    total = parts[0].copy()
    for z in range(1, splits):
        total = total + parts[z]            # float32, in order
    x = resid + total
    ref = plain.rms_norm(x, w, 1e-5)
    tol = 2e-6 * np.abs(ref).max() if dtype == torch.float32 else 2 ** -8 * np.abs(ref).max()
    r_dev = t32(resid)
    out = torch.empty(5, H, dtype=dtype, device=DEV)
    ops().add_rmsnorm(r_dev, t32(parts), t32(w), 1e-5, out)
    assert np.abs(out.float().cpu().numpy() - ref).max() <= tol
    assert np.abs(r_dev.cpu().numpy() - x).max() == 0.0
    rows = torch.tensor([4, 1], dtype=torch.int32, device=DEV)
    r_dev = t32(resid)
    out2 = torch.empty(2, H, dtype=dtype, device=DEV)
    ops().add_rmsnorm(r_dev, t32(parts), t32(w), 1e-5, out2, rows=rows)
    assert np.abs(out2.float().cpu().numpy() - ref[[4, 1]]).max() <= tol
    assert torch.equal(r_dev, t32(resid))


@pytest.mark.parametrize("H", [72, 1536, 3000])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_add_rmsnorm(H, dtype):
    rng = np.random.default_rng(H)
    resid = rng.standard_normal((7, H)).astype(np.float32) * 3
    delta = rng.standard_normal((7, H)).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    d_dev = t32(delta).to(dtype)
    x = resid + d_dev.float().cpu().numpy()
    ref = plain.rms_norm(x, w, 1e-5)
    r_dev = t32(resid)
    out = torch.empty(7, H, dtype=dtype, device=DEV)
    for wt in (t32(w), t32(w).to(torch.bfloat16)) if dtype == torch.bfloat16 else (t32(w),):
        r_dev = t32(resid)
        ops().add_rmsnorm(r_dev, d_dev, wt, 1e-5, out)
        refw = plain.rms_norm(x, wt.float().cpu().numpy(), 1e-5)
        tol = 2e-6 * np.abs(refw).max() if dtype == torch.float32 else 2 ** -8 * np.abs(refw).max()
        assert np.abs(out.float().cpu().numpy() - refw).max() <= tol
        assert np.abs(r_dev.cpu().numpy() - x).max() == 0.0       # residual updated in float32
    # gathered rows, no delta, residual untouched
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    r_dev = t32(resid)
    out3 = torch.empty(3, H, dtype=dtype, device=DEV)
    ops().add_rmsnorm(r_dev, None, t32(w), 1e-5, out3, rows=rows)
    ref3 = plain.rms_norm(resid[[6, 0, 3]], w, 1e-5)
    tol = 2e-6 * np.abs(ref3).max() if dtype == torch.float32 else 2 ** -8 * np.abs(ref3).max()
    assert np.abs(out3.float().cpu().numpy() - ref3).max() <= tol
    assert torch.equal(r_dev, t32(resid))
    assert ref.shape == (7, H)


@pytest.mark.parametrize("H", [64, 520, 1536, 3584, 5120, 8192])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_add_rmsnorm_many_rows(H, dtype):
    """More than 64 rows: one, two, four or eight warps per row (by the width), eight warps per CTA; a row
    count that does not fill the last CTA, rows gathered, the residual updated in float32."""
    n = 203
    rng = np.random.default_rng(H + 1)
    resid = rng.standard_normal((n, H)).astype(np.float32) * 3
    delta = rng.standard_normal((n, H)).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    d_dev = t32(delta).to(dtype)
    x = resid + d_dev.float().cpu().numpy()
    ref = plain.rms_norm(x, w, 1e-6)
    r_dev = t32(resid)
    out = torch.full((n, H), 7.0, dtype=dtype, device=DEV)
    ops().add_rmsnorm(r_dev, d_dev, t32(w), 1e-6, out)
    tol = 2e-6 * np.abs(ref).max() if dtype == torch.float32 else 2 ** -8 * np.abs(ref).max()
    assert np.abs(out.float().cpu().numpy() - ref).max() <= tol
    assert np.abs(r_dev.cpu().numpy() - x).max() == 0.0
    # gathered rows, no delta: the residual stays as it is
    pick = rng.permutation(n)[:100].astype(np.int32)
    r_dev = t32(resid)
    out2 = torch.empty(100, H, dtype=dtype, device=DEV)
    ops().add_rmsnorm(r_dev, None, t32(w), 1e-6, out2, rows=t32(pick))
    ref2 = plain.rms_norm(resid[pick], w, 1e-6)
    tol = 2e-6 * np.abs(ref2).max() if dtype == torch.float32 else 2 ** -8 * np.abs(ref2).max()
    assert np.abs(out2.float().cpu().numpy() - ref2).max() <= tol
    assert torch.equal(r_dev, t32(resid))


@pytest.mark.parametrize("shape", [(1, 50, 37), (5, 129, 200), (67, 96, 1000), (130, 300, 77)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gemm_simt(shape, dtype):
    M, N, K = shape
    rng = np.random.default_rng(M * N)
    x = t32(rng.standard_normal((M, K)).astype(np.float32)).to(dtype)
    w = t32(rng.standard_normal((N, K)).astype(np.float32)).to(dtype)
    b = t32(rng.standard_normal(N).astype(np.float32))
    ref = x.double().cpu() @ w.double().cpu().T + b.double().cpu()
    out = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops().gemm_simt(x, w, b, out)
    assert (out.double().cpu() - ref).abs().max() <= 1e-5 * ref.abs().max() + 1e-5
    # a strided input (a column slice of a wider buffer)
    wide = torch.zeros(M, K + 9, dtype=dtype, device=DEV)
    wide[:, 4:4 + K] = x
    out2 = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops().gemm_simt(wide[:, 4:4 + K], w, b, out2)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("shape", [(1, 50, 40), (3, 129, 200), (8, 96, 1000), (16, 2048, 1536), (17, 300, 72),
                                   (33, 1536, 8960), (64, 257, 96), (5, 151936, 64)])
@pytest.mark.parametrize("gated", [False, True])
def test_gemm_bf16_small(shape, gated):
    M, N, K = shape
    if gated and N % 2:
        N += 1
    rng = np.random.default_rng(M + N)
    x = t32(rng.standard_normal((M, K)).astype(np.float32)).to(torch.bfloat16)
    w = t32((rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)).to(torch.bfloat16)
    acc = x.double().cpu() @ w.double().cpu().T
    if gated:
        g, u = acc[:, 0::2], acc[:, 1::2]
        ref = g / (1 + torch.exp(-g)) * u
        out = torch.empty(M, N // 2, dtype=torch.bfloat16, device=DEV)
        ops().gemm_bf16_small(x, w, None, out, gated=True)
        assert (out.double().cpu() - ref).abs().max() <= 2 ** -8 * max(1.0, ref.abs().max()) + 1e-3
    else:
        b = t32(rng.standard_normal(N).astype(np.float32))
        ref = acc + b.double().cpu()
        out = torch.empty(M, N, dtype=torch.float32, device=DEV)
        ops().gemm_bf16_small(x, w, b, out)
        assert (out.double().cpu() - ref).abs().max() <= 2e-5 * max(1.0, ref.abs().max())
        outb = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        ops().gemm_bf16_small(x, w, b.to(torch.bfloat16), outb)
        assert (outb.double().cpu() - ref).abs().max() <= 2 ** -7 * max(1.0, ref.abs().max())
    with pytest.raises(Exception, match="multiples of 8"):
        ops().gemm_bf16_small(x[:, :K - 4].contiguous(), w[:, :K - 4].contiguous(), None,
                              torch.empty(M, N // 2 if gated else N, dtype=torch.float32, device=DEV), gated=gated)


@pytest.mark.parametrize("shape", [(1, 256, 1536), (8, 2048, 1536), (16, 17920, 1536), (5, 100, 72), (9, 50, 40),
                                   (17, 1536, 8960), (33, 300, 520), (64, 1536, 1536), (64, 151936, 64),
                                   (40, 2048, 1536), (3, 1000, 96), (2, 136, 4104), (100, 17920, 1536), (128, 1536, 8960),
                                   (200, 2048, 1536), (256, 300, 520), (65, 100, 72)])
@pytest.mark.parametrize("gated", [False, True])
def test_gemm_bf16_tc_few(shape, gated):
    """The few-rows tcgen05 kernel (features on the accumulator's lanes, K split over CTAs
    with an ordered reduction) against float64, with tails in N and K; twice in a row (the
    split counters reset themselves), and a row's result must not depend on the batch."""
    M, N, K = shape
    rng = np.random.default_rng(M + N + K)
    x = t32(rng.standard_normal((M, K)).astype(np.float32)).to(torch.bfloat16)
    w = t32((rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)).to(torch.bfloat16)
    acc = x.double().cpu() @ w.double().cpu().T
    if gated and M > 64 and ops().few_splits(N, K) > 1:
        with pytest.raises(Exception, match="left to the consumer"):
            ops().gemm_bf16_tc_few(x, w, None, torch.empty(M, N // 2, dtype=torch.bfloat16, device=DEV), gated=True)
    elif gated:
        g, u = acc[:, 0::2], acc[:, 1::2]
        ref = g / (1 + torch.exp(-g)) * u
        out = torch.full((M, N // 2), 7.0, dtype=torch.bfloat16, device=DEV)
        ops().gemm_bf16_tc_few(x, w, None, out, gated=True)
        ops().check_tc_status(DEV)
        assert (out.double().cpu() - ref).abs().max() <= 2 ** -8 * max(1.0, ref.abs().max()) + 1e-3
        again = torch.full_like(out, 3.0)
        ops().gemm_bf16_tc_few(x, w, None, again, gated=True)
        assert torch.equal(out, again)
    elif M > 64 and ops().few_splits(N, K) > 1:
        # more than 64 rows: a product whose K is cut leaves its slices to the consumer, or is refused
        b = t32(rng.standard_normal(N).astype(np.float32))
        ref = acc + b.double().cpu()
        S = ops().few_splits(N, K)
        parts = torch.full((S, M, N), 7.0, dtype=torch.float32, device=DEV)
        ops().gemm_bf16_tc_few(x, w, b, parts, defer=True)
        ops().check_tc_status(DEV)
        assert (parts.double().sum(0).cpu() - ref).abs().max() <= 3e-5 * max(1.0, ref.abs().max())
        alone = torch.empty(S, 1, N, dtype=torch.float32, device=DEV)
        ops().gemm_bf16_tc_few(x[M - 1:], w, b, alone, defer=True)
        assert torch.equal(alone[:, 0], parts[:, M - 1])        # the same bits as inside the batch
        with pytest.raises(Exception, match="left to the consumer"):
            ops().gemm_bf16_tc_few(x, w, b, torch.empty(M, N, dtype=torch.float32, device=DEV))
    else:
        b = t32(rng.standard_normal(N).astype(np.float32))
        ref = acc + b.double().cpu()
        out = torch.full((M, N), 7.0, dtype=torch.float32, device=DEV)
        ops().gemm_bf16_tc_few(x, w, b, out)
        ops().check_tc_status(DEV)
        assert (out.double().cpu() - ref).abs().max() <= 3e-5 * max(1.0, ref.abs().max())
        outb = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        ops().gemm_bf16_tc_few(x, w, None, outb)
        assert (outb.double().cpu() - acc).abs().max() <= 2 ** -7 * max(1.0, acc.abs().max())
        # a strided input (a column slice of a wider buffer, 16-byte aligned)
        wide = torch.zeros(M, K + 16, dtype=torch.bfloat16, device=DEV)
        wide[:, 8:8 + K] = x
        out2 = torch.empty(M, N, dtype=torch.float32, device=DEV)
        ops().gemm_bf16_tc_few(wide[:, 8:8 + K], w, b, out2)
        assert torch.equal(out, out2)
        # the last row alone: the same bits as inside the batch
        alone = torch.empty(1, N, dtype=torch.float32, device=DEV)
        ops().gemm_bf16_tc_few(x[M - 1:], w, b, alone)
        assert torch.equal(alone[0], out[M - 1])
        # the K slices' sums left to the consumer
        S = ops().few_splits(N, K)
        parts = torch.full((S, M, N), 7.0, dtype=torch.float32, device=DEV)
        ops().gemm_bf16_tc_few(x, w, b, parts, defer=True)
        assert (parts.double().sum(0).cpu() - ref).abs().max() <= 3e-5 * max(1.0, ref.abs().max())
        if S > 1 and K >= ops().DEFER_MIN_K and M <= ops().FEW_DEFER_M:
            assert torch.equal(ops().linear(x, w, b, partial_ok=True), parts)
    ops().check_tc_status(DEV)


@pytest.mark.parametrize("shape", [(256, 256, 64), (512, 512, 256), (300, 1000, 200), (1000, 520, 1096), (2048, 2048, 1536),
                                   (129, 40, 8), (2304, 4000, 328), (4096, 1536, 520)])
@pytest.mark.parametrize("gated", [False, True])
def test_gemm_bf16_tc_pairs_of_ctas(shape, gated):
    """The product by pairs of CTAs (tcgen05 cta_group::2, 256 x 256 tiles, two accumulators)
    against float64, with tails in M, N and K and more tiles than pairs; and the same bits as
    the single-CTA kernel, which sums K in the same order."""
    M, N, K = shape
    rng = np.random.default_rng(M + N + K)
    x = t32(rng.standard_normal((M, K)).astype(np.float32)).to(torch.bfloat16)
    w = t32((rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)).to(torch.bfloat16)
    acc = x.double().cpu() @ w.double().cpu().T
    if gated:
        g, u = acc[:, 0::2], acc[:, 1::2]
        ref = g / (1 + torch.exp(-g)) * u
        out = torch.full((M, N // 2), 7.0, dtype=torch.bfloat16, device=DEV)
        ops().gemm_bf16_tc_pair(x, w, None, out, gated=True)
        ops().check_tc_status(DEV)
        assert (out.double().cpu() - ref).abs().max() <= 2 ** -8 * max(1.0, ref.abs().max()) + 1e-3
    else:
        b = t32(rng.standard_normal(N).astype(np.float32))
        ref = acc + b.double().cpu()
        out = torch.full((M, N), 7.0, dtype=torch.float32, device=DEV)
        ops().gemm_bf16_tc_pair(x, w, b, out)
        ops().check_tc_status(DEV)
        assert (out.double().cpu() - ref).abs().max() <= 3e-5 * max(1.0, ref.abs().max())
        ops().set_gemm_pairs(False)
        try:
            single = torch.empty(M, N, dtype=torch.float32, device=DEV)
            ops().gemm_bf16_tc(x, w, b, single)
            unsplit = ops().gemm_tc_splits(M, N, K) == 1
        finally:
            ops().set_gemm_pairs(True)
        if unsplit:
            assert torch.equal(out, single)


@pytest.mark.parametrize("shape", [(128, 256, 64), (65, 32, 8), (200, 300, 136), (300, 1000, 96), (257, 96, 1000),
                                   (2048, 2048, 1536), (513, 1536, 8960), (130, 151936, 64), (1000, 48, 72),
                                   (64, 1536, 8960), (40, 2048, 1536), (17, 100, 520), (2304, 17920, 1536), (2048, 1536, 1536),
                                   (1000, 1100, 264)])
@pytest.mark.parametrize("gated", [False, True])
def test_gemm_bf16_tc(shape, gated):
    """TMA + tcgen05 kernel against float64, with tails in M, N and K."""
    M, N, K = shape
    rng = np.random.default_rng(M + N + K)
    x = t32(rng.standard_normal((M, K)).astype(np.float32)).to(torch.bfloat16)
    w = t32((rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)).to(torch.bfloat16)
    acc = x.double().cpu() @ w.double().cpu().T
    if gated:
        g, u = acc[:, 0::2], acc[:, 1::2]
        ref = g / (1 + torch.exp(-g)) * u
        out = torch.full((M, N // 2), 7.0, dtype=torch.bfloat16, device=DEV)
        ops().gemm_bf16_tc(x, w, None, out, gated=True)
        ops().check_tc_status(DEV)
        assert (out.double().cpu() - ref).abs().max() <= 2 ** -8 * max(1.0, ref.abs().max()) + 1e-3
    else:
        b = t32(rng.standard_normal(N).astype(np.float32))
        ref = acc + b.double().cpu()
        out = torch.full((M, N), 7.0, dtype=torch.float32, device=DEV)
        ops().gemm_bf16_tc(x, w, b, out)
        ops().check_tc_status(DEV)
        assert (out.double().cpu() - ref).abs().max() <= 3e-5 * max(1.0, ref.abs().max())
        outb = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        ops().gemm_bf16_tc(x, w, None, outb)
        assert (outb.double().cpu() - acc).abs().max() <= 2 ** -7 * max(1.0, acc.abs().max())
        # a strided input (a column slice of a wider buffer, 16-byte aligned)
        wide = torch.zeros(M, K + 16, dtype=torch.bfloat16, device=DEV)
        wide[:, 8:8 + K] = x
        out2 = torch.empty(M, N, dtype=torch.float32, device=DEV)
        ops().gemm_bf16_tc(wide[:, 8:8 + K], w, b, out2)
        assert torch.equal(out, out2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rows_do_not_depend_on_batch(dtype):
    """A row's product is the same alone and inside a larger batch (bitwise)."""
    rng = np.random.default_rng(1)
    x = t32(rng.standard_normal((70, 160)).astype(np.float32)).to(dtype)
    w = t32(rng.standard_normal((90, 160)).astype(np.float32)).to(dtype)
    full = ops().linear(x, w)
    for r in (0, 13, 69):
        assert torch.equal(ops().linear(x[r:r + 1].contiguous(), w)[0], full[r])
    if dtype == torch.bfloat16:     # the weight-streaming kernel: 1, 9, 33 and 64 rows agree bitwise
        big = torch.empty(64, 90, dtype=dtype, device=DEV)
        ops().gemm_bf16_small(x[:64].contiguous(), w, None, big)
        for m in (1, 9, 33):
            part = torch.empty(m, 90, dtype=dtype, device=DEV)
            ops().gemm_bf16_small(x[:m].contiguous(), w, None, part)
            assert torch.equal(part, big[:m])
        # and the TMA/tcgen05 kernel: a row alone in its tile or among 69 others
        tc_full = torch.empty(70, 90, dtype=dtype, device=DEV)
        ops().gemm_bf16_tc(x, w, None, tc_full)
        tc_part = torch.empty(17, 90, dtype=dtype, device=DEV)
        ops().gemm_bf16_tc(x[40:57].contiguous(), w, None, tc_part)
        assert torch.equal(tc_part, tc_full[40:57])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_silu_mul(dtype):
    rng = np.random.default_rng(2)
    gu = t32(rng.standard_normal((9, 2 * 77)).astype(np.float32) * 4).to(dtype)
    out = torch.empty(9, 77, dtype=dtype, device=DEV)
    ops().silu_mul(gu, out)
    g = gu.float().cpu().numpy()
    ref = plain.swiglu(g[:, 0::2], g[:, 1::2])
    tol = 1e-6 if dtype == torch.float32 else 2 ** -8
    assert np.abs(out.float().cpu().numpy() - ref).max() <= tol * max(1, np.abs(ref).max())


def paged_setup(rng, lens, nkv, hd, page_size, dtype, shuffle=True):
    """Random keys/values for requests of the given lengths laid into shuffled pages."""
    B = len(lens)
    blocks = [-(-n // page_size) for n in lens]
    total = sum(blocks) + 3
    order = rng.permutation(total) if shuffle else np.arange(total)
    kc = torch.zeros(total, nkv, page_size, hd, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    bt = np.full((B, max(blocks)), -1, np.int32)
    ks, vs = [], []
    nxt = 0
    for b, n in enumerate(lens):
        k = torch.from_numpy(rng.standard_normal((n, nkv, hd)).astype(np.float32)).to(dtype)
        v = torch.from_numpy(rng.standard_normal((n, nkv, hd)).astype(np.float32)).to(dtype)
        ks.append(k.float().numpy()); vs.append(v.float().numpy())
        for j in range(blocks[b]):
            p = int(order[nxt]); nxt += 1
            bt[b, j] = p
            lo, hi = j * page_size, min(n, (j + 1) * page_size)
            kc[p, :, :hi - lo] = k[lo:hi].permute(1, 0, 2).to(DEV)
            vc[p, :, :hi - lo] = v[lo:hi].permute(1, 0, 2).to(DEV)
    return kc, vc, t32(bt), ks, vs


def attention_reference(q_rows, ks, vs, reqs, poss, nh, nkv, hd, window, scale):
    """Plain attention of single rows: row i belongs to request reqs[i] at position poss[i]."""
    out = np.zeros((len(reqs), nh * hd), np.float32)
    for i, (b, p) in enumerate(zip(reqs, poss)):
        first = max(0, p - window + 1) if window else 0
        k = ks[b][first:p + 1].astype(np.float64)
        v = vs[b][first:p + 1].astype(np.float64)
        for h in range(nh):
            g = h // (nh // nkv)
            s = (k[:, g] @ q_rows[i, h * hd:(h + 1) * hd].astype(np.float64)) * scale
            e = np.exp(s - s.max())
            out[i, h * hd:(h + 1) * hd] = (e / e.sum()) @ v[:, g]
    return out


@pytest.mark.parametrize("nh,nkv,hd,page", [(4, 2, 16, 16), (3, 1, 32, 16), (7, 7, 48, 8), (12, 2, 128, 16),
                                            (5, 1, 80, 32), (6, 3, 112, 16)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 37])
def test_attention(nh, nkv, hd, page, dtype, window):
    rng = np.random.default_rng(nh * 100 + hd)
    lens = [1, 130, 47, 64]
    kc, vc, bt, ks, vs = paged_setup(rng, lens, nkv, hd, page, dtype)
    # rows: a whole request, the tail of another, single last tokens of the rest
    reqs = [0] + [1] * 30 + [2] * 47 + [3]
    poss = [0] + list(range(100, 130)) + list(range(47)) + [63]
    T = len(reqs)
    q = torch.from_numpy(rng.standard_normal((T, nh * hd)).astype(np.float32)).to(dtype).to(DEV)
    out = torch.empty(T, nh * hd, dtype=dtype, device=DEV)
    scale = 1.0 / np.sqrt(hd)
    ref = attention_reference(q.float().cpu().numpy(), ks, vs, reqs, poss, nh, nkv, hd, window, scale)
    # bfloat16: the output is rounded to 8 bits (relative 2^-9, taken as 2^-8), and the
    # tensor-core kernels also round the probabilities to bfloat16 before P V (absolute 2^-8
    # for values of unit spread)
    tol = 2e-5 if dtype == torch.float32 else 2 ** -8 * np.abs(ref) + 2 ** -8
    q_lens = [1, 30, 47, 1]
    hints = dict(cu_q=t32(np.asarray([0, 1, 31, 78, 79], np.int32)), kv_lens=t32(np.asarray(lens, np.int32)),
                 q_lens=q_lens, max_kv_len=max(lens))
    for force_simple in (True, False):       # the plain kernel, then the one the engine picks
        out.zero_()
        ops().attention_rows(q, out, kc, vc, bt, t32(np.asarray(reqs, np.int32)), t32(np.asarray(poss, np.int32)),
                             nh, nkv, hd, page, window, scale, force_simple=force_simple, **hints)
        assert np.all(np.abs(out.float().cpu().numpy() - ref) <= tol), force_simple


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_finds_a_far_key(dtype):
    """One key among 700 is made to stand out (its score dominates): the output must be
    that key's value.  Random weights alone would hide a kernel that skips far keys, a
    page's edge or the window's first position."""
    nh, nkv, hd, page = 4, 2, 64, 16
    rng = np.random.default_rng(9)
    n = 700
    scale = 1.0 / np.sqrt(hd)
    for target, window in [(3, None), (15, None), (16, None), (352, None), (n - 200, 200), (n - 201, 200)]:
        kc, vc, bt, ks, vs = paged_setup(rng, [n], nkv, hd, page, dtype, shuffle=True)
        q = rng.standard_normal((1, nh * hd)).astype(np.float32)
        # make key[target] of every kv head parallel to the queries of its group, and long
        p = int(bt[0, target // page].item()); o = target % page
        for g in range(nkv):
            qg = q[0, g * (nh // nkv) * hd:(g * (nh // nkv) + 1) * hd]
            for h in range(g * (nh // nkv), (g + 1) * (nh // nkv)):
                q[0, h * hd:(h + 1) * hd] = qg
            kc[p, g, o] = torch.from_numpy(qg * 40 / np.linalg.norm(qg)).to(dtype).to(DEV) * 4
            ks[0][target, g] = kc[p, g, o].float().cpu().numpy()
        qd = t32(q).to(dtype)
        out = torch.empty(1, nh * hd, dtype=dtype, device=DEV)
        ops().attention_rows(qd, out, kc, vc, bt, t32(np.zeros(1, np.int32)), t32(np.asarray([n - 1], np.int32)),
                             nh, nkv, hd, page, window, scale, cu_q=t32(np.asarray([0, 1], np.int32)),
                             kv_lens=t32(np.asarray([n], np.int32)), q_lens=[1], max_kv_len=n)
        ref = attention_reference(qd.float().cpu().numpy(), ks, vs, [0], [n - 1], nh, nkv, hd, window, scale)
        got = out.float().cpu().numpy()
        assert np.abs(got - ref).max() <= (2e-5 if dtype == torch.float32 else 2 ** -6), (target, window)
        inside = window is None or target > n - 1 - window
        for h in range(nh):
            hit = np.abs(got[0, h * hd:(h + 1) * hd] - vs[0][target, h // (nh // nkv)]).max() < 0.05
            assert hit == inside, (target, window, h)


@pytest.mark.parametrize("nh,nkv,hd,page", [(12, 2, 128, 16), (4, 1, 64, 8), (8, 8, 128, 64), (6, 2, 64, 128),
                                            (16, 1, 128, 256), (3, 1, 192, 32), (2, 1, 256, 16)])
@pytest.mark.parametrize("window", [None, 200])
@pytest.mark.parametrize("cluster,two_tiles", [(0, True), (0, False), (2, False), (8, False)])
def test_attention_prompt_portions_tensor_memory(nh, nkv, hd, page, window, cluster, two_tiles):
    """Prompt portions through the tcgen05 kernels (S and O in tensor memory, P fed back from
    it): whole prompts and tails that start inside a key tile, several key tiles, row tiles
    that end inside a token group, a window that begins inside a tile; with two row tiles per
    CTA sharing every fetched key tile (an odd number of row tiles leaves the last CTA one), with
    one, and with the key tiles of a row tile split over 2 or 8 CTAs of a cluster (some of them
    left without a tile) and merged through distributed shared memory."""
    rng = np.random.default_rng(nh + hd + page)
    lens = [300, 700, 129, 64]
    q_lens = [300, 257, 20, 64]
    kc, vc, bt, ks, vs = paged_setup(rng, lens, nkv, hd, page, torch.bfloat16)
    reqs, poss = [], []
    for b, (n, ql) in enumerate(zip(lens, q_lens)):
        reqs += [b] * ql
        poss += list(range(n - ql, n))
    T = len(reqs)
    q = torch.from_numpy(rng.standard_normal((T, nh * hd)).astype(np.float32)).to(torch.bfloat16).to(DEV)
    scale = 1.0 / np.sqrt(hd)
    cu = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    out = torch.zeros(T, nh * hd, dtype=torch.bfloat16, device=DEV)
    ops().set_attention_tc_cluster(hd, cluster)
    ops().set_attention_tc_two_tiles(hd, two_tiles)
    try:
        ops().attention_rows(q, out, kc, vc, bt, t32(np.asarray(reqs, np.int32)), t32(np.asarray(poss, np.int32)),
                             nh, nkv, hd, page, window, scale, cu_q=t32(cu), kv_lens=t32(np.asarray(lens, np.int32)),
                             q_lens=q_lens, max_kv_len=max(lens))
        ops().check_tc_status(DEV)
    finally:
        ops().set_attention_tc_cluster(hd, 0)
        ops().set_attention_tc_two_tiles(hd, None)
    ref = attention_reference(q.float().cpu().numpy(), ks, vs, reqs, poss, nh, nkv, hd, window, scale)
    tol = 2 ** -8 * np.abs(ref) + 2 ** -8
    err = np.abs(out.float().cpu().numpy() - ref)
    assert np.all(err <= tol), (float(err.max()), np.argwhere(err > tol)[:5].tolist())


@pytest.mark.parametrize("window", [None, 700])
def test_attention_long_prompt_takes_two_row_tiles_per_cta(window):
    """A prompt long enough that pairs of row tiles still fill the GPU (192 CTAs of 256 rows here)
    goes to the kernel with two row tiles per CTA by itself; a sample of its rows is compared with
    the plain attention, all of them with the kernel that gives every row tile a CTA of its own."""
    nh, nkv, hd, page, n = 16, 8, 64, 16, 3000
    rng = np.random.default_rng(77)
    kc, vc, bt, ks, vs = paged_setup(rng, [n], nkv, hd, page, torch.bfloat16)
    q = torch.from_numpy(rng.standard_normal((n, nh * hd)).astype(np.float32)).to(torch.bfloat16).to(DEV)
    scale = 1.0 / np.sqrt(hd)
    args = (kc, vc, bt, t32(np.zeros(n, np.int32)), t32(np.arange(n, dtype=np.int32)), nh, nkv, hd, page, window, scale)
    kw = dict(cu_q=t32(np.asarray([0, n], np.int32)), kv_lens=t32(np.asarray([n], np.int32)), q_lens=[n], max_kv_len=n)
    outs = {}
    try:
        for mode in (None, False):
            ops().set_attention_tc_two_tiles(hd, mode)
            before = ops().total_launch_count()
            outs[mode] = torch.zeros(n, nh * hd, dtype=torch.bfloat16, device=DEV)
            ops().attention_rows(q, outs[mode], *args, **kw)
            ops().check_tc_status(DEV)
            assert ops().total_launch_count() == before + 1
    finally:
        ops().set_attention_tc_two_tiles(hd, None)
    rows = np.unique(np.concatenate([rng.integers(0, n, 40), [0, 1, 127, 128, 255, 256, 699, 700, 701, n - 1]]))
    ref = attention_reference(q.float().cpu().numpy()[rows], ks, vs, [0] * len(rows), rows.tolist(), nh, nkv, hd, window, scale)
    got = outs[None].float().cpu().numpy()
    tol = 2 ** -8 * np.abs(ref) + 2 ** -8
    err = np.abs(got[rows] - ref)
    assert np.all(err <= tol), (float(err.max()), np.argwhere(err > tol)[:5].tolist())
    # the two kernels order their sums differently and move the exponent's reference at different tiles
    assert float((got - outs[False].float().cpu().numpy()).max()) <= 2 ** -6


@pytest.mark.parametrize("nh,nkv,hd,K,page", [(12, 2, 128, 1536, 16), (4, 2, 16, 64, 16), (3, 1, 32, 96, 8), (5, 5, 48, 200, 32)])
@pytest.mark.parametrize("T", [1, 7, 16])
def test_qkv_product_with_rotation_and_cache_write(nh, nkv, hd, K, page, T):
    """The decode product that rotates and writes the cache in its epilogue gives the bits of the
    product followed by the rotation kernel."""
    rng = np.random.default_rng(nh + hd + T)
    N = (nh + 2 * nkv) * hd
    x = t32(rng.standard_normal((T, K)).astype(np.float32)).to(torch.bfloat16)
    w = t32((rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)).to(torch.bfloat16)
    b = t32(rng.standard_normal(N).astype(np.float32))
    max_pos = 300
    ang = rng.uniform(0, 6.28, size=(max_pos, hd // 2)).astype(np.float32)
    cos_sin = t32(np.stack([np.cos(ang), np.sin(ang)], axis=-1).astype(np.float32))
    positions = t32(rng.integers(0, max_pos, size=T).astype(np.int32))
    pages = 40
    slots_np = rng.permutation(pages * page)[:T].astype(np.int32)
    if T > 2:
        slots_np[1] = -1                               # a row that writes nothing
    slots = t32(slots_np)
    kc = torch.zeros(pages, nkv, page, hd, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    q = ops().qkv_rope_small(x, w, b, positions, cos_sin, slots, kc, vc, nh, nkv, hd, page)
    qkv = torch.empty(T, N, dtype=torch.bfloat16, device=DEV)
    ops().gemm_bf16_small(x, w, b, qkv)               # the same kernel family: the same order of summation
    kc2, vc2 = torch.zeros_like(kc), torch.zeros_like(vc)
    ops().rope_kv_write(qkv, positions, cos_sin, slots, kc2, vc2, nh, nkv, hd, hd, page)
    assert torch.equal(q, qkv[:, :nh * hd])
    assert torch.equal(kc, kc2) and torch.equal(vc, vc2)


@pytest.mark.parametrize("split", [128, 192, 256, 512, 1024, 2048, 0])
@pytest.mark.parametrize("nh,nkv,hd,page", [(12, 2, 128, 64), (3, 1, 32, 16), (14, 2, 64, 8), (4, 2, 16, 2)])
def test_decode_attention_split_sizes(split, nh, nkv, hd, page):
    """The decode kernel at each of its split sizes (pages of two positions cap the split at 512): lengths
    around tile (64) and split edges, two-token tails, and windows that begin inside a tile and inside a split."""
    rng = np.random.default_rng(split + hd)
    lens = [1, 63, 64, 65, 129, 511, 512, 513, 700, 1300, 2049, 2500]
    dtype = torch.bfloat16
    kc, vc, bt, ks, vs = paged_setup(rng, lens, nkv, hd, page, dtype)
    q_lens = [1, 1, 1, 2, 1, 1, 2, 1, 1, 1, 2, 1] if (nh // nkv) * 2 <= 16 else [1] * len(lens)
    reqs, poss = [], []
    for b, (n, ql) in enumerate(zip(lens, q_lens)):
        ql = min(ql, n)
        q_lens[b] = ql
        reqs += [b] * ql
        poss += list(range(n - ql, n))
    T = len(reqs)
    q = torch.from_numpy(rng.standard_normal((T, nh * hd)).astype(np.float32)).to(dtype).to(DEV)
    scale = 1.0 / np.sqrt(hd)
    cu = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    ops().set_attention_split(hd, split)
    try:
        for window in (None, 100, 333, 640):
            out = torch.zeros(T, nh * hd, dtype=dtype, device=DEV)
            ops().attention_rows(q, out, kc, vc, bt, t32(np.asarray(reqs, np.int32)), t32(np.asarray(poss, np.int32)),
                                 nh, nkv, hd, page, window, scale, cu_q=t32(cu), kv_lens=t32(np.asarray(lens, np.int32)),
                                 q_lens=q_lens, max_kv_len=max(lens))
            ref = attention_reference(q.float().cpu().numpy(), ks, vs, reqs, poss, nh, nkv, hd, window, scale)
            tol = 2 ** -8 * np.abs(ref) + 2 ** -8
            assert np.all(np.abs(out.float().cpu().numpy() - ref) <= tol), window
    finally:
        ops().set_attention_split(hd, 0)


@pytest.mark.parametrize("nh,nkv,hd,rot", [(4, 2, 16, 16), (3, 1, 32, 32), (5, 5, 48, 48), (2, 1, 64, 32)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rope_kv_write(nh, nkv, hd, rot, dtype):
    from coheryn_ai_studio_b200.parts.base import Runtime
    from coheryn_ai_studio_b200.parts.position import RotateHalfRope
    rng = np.random.default_rng(hd)
    theta, T, page = 1e6, 11, 8
    pos_part = RotateHalfRope(Runtime(dtype, torch.device(DEV)), hd, rot, theta, 600)
    positions = np.array([0, 1, 7, 511, 300, 2, 3, 4, 5, 6, 599], np.int32)
    width = (nh + 2 * nkv) * hd
    qkv = torch.from_numpy(rng.standard_normal((T, width)).astype(np.float32)).to(dtype)
    src = qkv.float().numpy().copy()
    dev = qkv.to(DEV)
    kc = torch.zeros(5, nkv, page, hd, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    slots = rng.permutation(5 * page)[:T].astype(np.int32)
    ops().rope_kv_write(dev, t32(positions), pos_part.cos_sin(), t32(slots), kc, vc, nh, nkv, hd, rot, page)
    got = dev.float().cpu().numpy()
    tol = 3e-6 if dtype == torch.float32 else 2 ** -7
    def rotated(x):  # x: [T, heads*hd]; rotate the first ``rot`` of each head
        h = x.reshape(T, -1, hd).copy()
        part = plain.rope(h[:, :, :rot].reshape(T, -1), positions, rot, theta).reshape(T, -1, rot)
        h[:, :, :rot] = part
        return h.reshape(T, -1)
    q_ref = rotated(src[:, :nh * hd])
    k_ref = rotated(src[:, nh * hd:(nh + nkv) * hd]).reshape(T, nkv, hd)
    v_ref = src[:, (nh + nkv) * hd:].reshape(T, nkv, hd)
    scale = max(1.0, np.abs(q_ref).max())
    assert np.abs(got[:, :nh * hd] - q_ref).max() <= tol * scale
    for t in range(T):
        p, o = divmod(int(slots[t]), page)
        assert np.abs(kc[p, :, o].float().cpu().numpy() - k_ref[t]).max() <= tol * scale
        assert np.array_equal(vc[p, :, o].float().cpu().numpy(), v_ref[t])


def test_rope_table_matches_reference_fixture():
    """The engine's own rotation (table + kernel) against the reference's RoPE fixture."""
    import json, os
    from coheryn_ai_studio_b200.parts.base import Runtime
    from coheryn_ai_studio_b200.parts.position import RotateHalfRope
    fx = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_rope.json")))
    for case in fx["cases"]:
        hd, p = case["head_dim"], case["position"]
        part = RotateHalfRope(Runtime(torch.float32, torch.device(DEV)), hd, hd, float(case["base"]), 512)
        x = t32(np.asarray(case["input"], np.float32)[None, :])
        heads = x.shape[1] // hd
        ops().rope_kv_write(x, t32(np.asarray([p], np.int32)), part.cos_sin(), None, None, None,
                            heads, 0, hd, hd, 16)
        ref = np.asarray(case["output"], np.float64)
        assert np.all(np.abs(x.cpu().numpy()[0] - ref) <= 2e-6 + 2e-6 * np.abs(ref)), (hd, p)


def test_argmax_first_maximum():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((5, 1000)).astype(np.float32)
    x[0, 17] = x[0, 900] = 9.0           # tie: lowest id wins
    x[1, 999] = 50.0
    x[2, :] = 0.0                        # all equal -> 0
    lg = t32(x)
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops().argmax(lg, out, status)
    assert out.tolist() == [17, 999, 0, int(x[3].argmax()), int(x[4].argmax())] and status.item() == 0
    lg[3, 5] = float("nan")
    ops().argmax(lg, out, status)
    assert status.item() == 2


def test_argmax_wide_rows_use_many_blocks():
    rng = np.random.default_rng(4)
    x = rng.standard_normal((9, 151936)).astype(np.float32)
    x[0, 4095] = x[0, 4096] = x[0, 151935] = 99.0        # ties across pieces: lowest id wins
    x[1, 151935] = 77.0
    out = torch.empty(9, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops().argmax(t32(x), out, status)
    assert out.tolist() == [4095, 151935] + [int(r.argmax()) for r in x[2:]] and status.item() == 0


@pytest.mark.parametrize("V", [5, 1000, 151936])
def test_sample_follows_reference_order(V):
    """The device sampler picks what the plain float64 sampler picks, for the same draws."""
    rng = np.random.default_rng(V)
    settings = [(0.8, 0, 1.0), (1.0, 5, 1.0), (0.7, 0, 0.9), (1.5, 50, 0.95), (0.3, 2, 0.5), (2.0, 0, 1.0)]
    R = len(settings)
    logits = (rng.standard_normal((R, V)) * 3).astype(np.float32)
    logits[1, :4] = logits[1].max() + 1.0       # ties at the top: ranked by id
    lg = t32(logits)
    samplers = [plain.PlainSampler(temperature=t, top_k=min(k, V), top_p=p, seed=100 + i)
                for i, (t, k, p) in enumerate(settings)]
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    temp = t32(np.asarray([s[0] for s in settings], np.float32))
    topk = t32(np.asarray([min(s[1], V) for s in settings], np.int32))
    topp = t32(np.asarray([s[2] for s in settings], np.float32))
    draws = 12 if V > 10000 else 40
    twins = [plain.PlainSampler(temperature=t, top_k=min(k, V), top_p=p, seed=100 + i)
             for i, (t, k, p) in enumerate(settings)]
    for _ in range(draws):
        u = np.asarray([tw.random() for tw in twins], np.float64)
        ops().sample(lg, temp, topk, topp, t32(u), out, status)
        want = [s.sample(logits[i]) for i, s in enumerate(samplers)]
        assert out.tolist() == want
    assert status.item() == 0




# ------------------------------------------------------------------ seeded weights, row moves, status
def test_seeded_fill_on_the_device_equals_numpy_bit_for_bit():
    """The CUDA generator, the host runtime's and the numpy restatement of the plain implementation
    give the same bits: float32 and bfloat16, a start in the middle of a tensor, an index beyond 2^32."""
    import plain_random as pr
    from coheryn_ai_studio_b200.weights.seeded import seeded_tensor
    name = "model.layers.1.mlp.down_proj.weight"
    for seed, first, n, mean, dev in [(11, 0, 300_001, 0.0, 0.02), (1, 2 ** 32 + 7, 8191, 1.0, 0.01), (2 ** 64 - 1, 5, 2048, 0.0, 0.1)]:
        ref = pr.values(pr.tensor_key(seed, name), np.arange(first, first + n, dtype=np.uint64), mean, dev)
        got = seeded_tensor(seed, name, (n,), mean, dev, device=DEV, first=first)
        host = seeded_tensor(seed, name, (n,), mean, dev, device="cpu", first=first)
        assert np.array_equal(got.cpu().numpy().view(np.uint32), ref.view(np.uint32))
        assert torch.equal(got.cpu(), host)
        got16 = seeded_tensor(seed, name, (n,), mean, dev, dtype=torch.bfloat16, device=DEV, first=first)
        assert np.array_equal(got16.float().cpu().numpy().view(np.uint32), pr.round_bf16(ref).view(np.uint32))


def test_random_model_on_the_device_equals_the_folder(tmp_path):
    """One seed, one model: the folder written on the host and the model made on the device hold
    the same values (so what a benchmark times can be checked against the plain implementation)."""
    import tiny
    from coheryn_ai_studio_b200.engine import load_model, random_model_on_device, write_random_model
    from coheryn_ai_studio_b200.weights import InitPolicy
    pol = InitPolicy(0.05, 0.1, 0.02)
    folder = str(tmp_path / "m")
    write_random_model(folder, tiny.TINY_B, 9, pol)
    a = load_model(folder, "bfloat16")[1]
    b = random_model_on_device(tiny.TINY_B, 9, "bfloat16", policy=pol)
    assert torch.equal(a.embedding, b.embedding) and torch.equal(a.head, b.head)
    for la, lb in zip(a.layers, b.layers):
        assert torch.equal(la.mixer.w_qkv, lb.mixer.w_qkv) and torch.equal(la.mixer.b_qkv.float(), lb.mixer.b_qkv.float())
        assert torch.equal(la.feed_forward.w_gate_up, lb.feed_forward.w_gate_up)
        assert torch.equal(la.mixer_norm.weight.float(), lb.mixer_norm.weight.float())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int32])
def test_gather_scatter_rows(dtype):
    rng = np.random.default_rng(2)
    for T, H in [(37, 72), (9, 5), (64, 1)]:
        src = torch.from_numpy(rng.integers(-1000, 1000, (T, H)).astype(np.float32)).to(dtype).to(DEV)
        rows = torch.from_numpy(rng.integers(0, T, 21).astype(np.int32)).to(DEV)
        assert torch.equal(ops().gather_rows(src, rows), src[rows.long()])
        wide = torch.zeros((T, H + 8), dtype=dtype, device=DEV)
        wide[:, :H] = src
        assert torch.equal(ops().gather_rows(wide[:, :H], rows), src[rows.long()])      # a column slice: strided rows
    vec = torch.arange(50, dtype=torch.int32, device=DEV)
    rows = torch.tensor([49, 0, 7], dtype=torch.int32, device=DEV)
    assert ops().gather_rows(vec, rows).tolist() == [49, 0, 7]
    out = torch.full((50,), -1, dtype=torch.int32, device=DEV)
    ops().scatter_words(torch.tensor([5, 6, 7], dtype=torch.int32, device=DEV), rows, out)
    assert out[49].item() == 5 and out[0].item() == 6 and out[7].item() == 7 and int((out == -1).sum()) == 47


def test_scale_add_bias_and_embedding_scale():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((5, 1003)).astype(np.float32)
    b = rng.standard_normal(1003).astype(np.float32)
    for scale, bias in [(0.5, b), (None, b), (3.0, None)]:
        t = t32(x)
        ops().scale_add_bias(t, scale, t32(bias) if bias is not None else None)
        want = x * np.float32(1.0 if scale is None else scale) + (bias if bias is not None else 0)
        assert np.abs(t.cpu().numpy() - want).max() <= 1e-6
    table = t32(rng.standard_normal((30, 24)).astype(np.float32))
    ids = torch.tensor([3, 29, 0], dtype=torch.int32, device=DEV)
    out = torch.empty((3, 24), dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops().embed_gather(table, ids, out, status, scale=1.75)
    assert torch.equal(out, table[ids.long()] * 1.75) and status.item() == 0


def test_unbuilt_gated_activation_is_refused_by_name():
    with pytest.raises(ops().KernelError, match="gelu"):
        ops().gated_activation_code("gelu")
    x = torch.zeros((4, 64), dtype=torch.bfloat16, device=DEV)
    w = torch.zeros((32, 64), dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ops().KernelError, match="relu2"):
        ops().gated_linear(x, w, "relu2")
    assert ops().gated_linear(x, w, "silu").shape == (4, 16)


def test_a_wait_that_runs_out_becomes_an_error_on_the_host(tmp_path):
    """A bounded wait that gives up leaves a code in the status word of the tensor-core kernels; the
    step function, the replay program's check and the engine's sampling path all read that word and
    raise.  The wait here is the self-test kernel's: a barrier that nothing arrives on, a few hundred
    tries, nothing in flight when it gives up."""
    import tiny
    from coheryn_ai_studio_b200.cache import CacheManager
    from coheryn_ai_studio_b200.engine import Engine, StepEntry, StepRunner, load_model
    dev = torch.device(DEV)
    ops().check_tc_status(dev)                                   # clean before
    ops().selftest_bounded_wait(dev, tries=300)
    with pytest.raises(ops().KernelError, match="bounded wait"):
        ops().check_tc_status(dev)
    ops().check_tc_status(dev)                                   # reading it cleared it
    folder = tiny.make_folder(tmp_path, "A")
    model = load_model(folder, "bfloat16")[1]
    cache = CacheManager(model.cache_requirements(), [None] * len(model.spec.schedule), torch.bfloat16, dev,
                         page_size=16, num_pages=8, max_requests=2, prefix_reuse=False)
    runner = StepRunner(model, cache)
    cache.admit("r")
    runner.step([StepEntry("r", [1, 2, 3], [2])])
    runner.check_status()
    ops().selftest_bounded_wait(dev, tries=200)
    runner.step([StepEntry("r", [4], [0])])
    with pytest.raises(RuntimeError, match="bounded wait"):
        runner.check_status()
    runner.check_status()
    eng = Engine(model, dtype="bfloat16", context=64, max_num_seqs=2)
    eng.add_request([5, 6, 7], max_tokens=4)
    eng.step()
    ops().selftest_bounded_wait(dev, tries=200)
    with pytest.raises(RuntimeError, match="bounded wait"):
        while eng.has_work():
            eng.step()
    assert int(ops().tc_status(dev).item()) == 0


def test_device_sampler_on_the_reference_fixture():
    """The reference's sampling fixture (fixtures/constraints/sampling-v2.json: a greedy tie, a seeded
    masked top-k/top-p case, negative penalties, the largest seed) through the DEVICE sampler.  The
    engine has no mask option; a masked entry is presented as a logit far below every other, which
    the kernels rank last and give no mass."""
    import json
    import os
    from coheryn_ai_studio_b200.sampling import DeviceSampler, RequestSampler, SamplingParams
    fx = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_sampling_v2.json")))
    sampler = DeviceSampler(torch.device(DEV))
    for case in fx["cases"]:
        params = SamplingParams(**case["settings"], **case["penalties"])
        rs = RequestSampler(params, case["history"])
        base = np.asarray(case["logits"], np.float32)
        base[~np.asarray(case["allowed"], bool)] = np.float32(-3.0e38)
        for expected in case["expected_ids"]:
            logits = torch.from_numpy(base.copy()).to(DEV)[None, :]
            assert sampler.sample(logits, [rs]) == [expected], case["id"]


@pytest.mark.parametrize("nh,nkv,hd,page,H", [(12, 2, 128, 16, 1536), (4, 2, 16, 16, 64), (3, 1, 32, 8, 100), (16, 1, 64, 16, 200),
                                              (6, 3, 112, 32, 264)])
@pytest.mark.parametrize("window", [None, 150])
def test_decode_attention_with_the_projection_merged(nh, nkv, hd, page, H, window):
    """attn_merge_oproj: decode attention of one token per request with the splits merged inside the
    output projection's kernel.  The sum of the heads' parts equals plain attention times the output
    matrix; requests of one key, of a split's edge (128, 129) and of many splits; widths that are no
    multiple of the 128-feature tile; a bias."""
    from types import SimpleNamespace
    rng = np.random.default_rng(nh * 7 + hd)
    lens = [1, 128, 129, 700, 64, 333, 2, 513, 40]
    B = len(lens)
    kc, vc, bt, ks, vs = paged_setup(rng, lens, nkv, hd, page, torch.bfloat16, shuffle=True)
    q = torch.from_numpy(rng.standard_normal((B, nh * hd)).astype(np.float32)).to(torch.bfloat16).to(DEV)
    w = torch.from_numpy((rng.standard_normal((H, nh * hd)) * 0.05).astype(np.float32)).to(torch.bfloat16).to(DEV)
    bias = torch.from_numpy(rng.standard_normal(H).astype(np.float32)).to(DEV)
    scale = 1.0 / np.sqrt(hd)
    step = SimpleNamespace(block_tables=[bt], cu_q=t32(np.arange(B + 1, dtype=np.int32)), kv_lens=t32(np.asarray(lens, np.int32)),
                           num_requests=B, max_q_len=1, max_kv_len=max(lens), prior_positions_settled=True)
    assert ops().attention_oproj_ok(q, w, step, nh, nkv, hd)
    for b_o in (None, bias):
        parts = ops().attention_oproj(q, kc, vc, step, 0, nh, nkv, hd, page, window, scale, w, b_o)
        assert parts.shape == (nh, B, H)
        attended = attention_reference(q.float().cpu().numpy(), ks, vs, list(range(B)), [n - 1 for n in lens], nh, nkv, hd,
                                       window, scale)
        rounded = torch.from_numpy(attended).to(torch.bfloat16).float().numpy()       # the kernel rounds the merged rows
        ref = plain.linear(rounded, w.float().cpu().numpy(), None if b_o is None else bias.cpu().numpy())
        got = parts.sum(0).cpu().numpy()
        # merged rows rounded to 8 bits of mantissa before the product: relative 2^-8 of each row's terms
        tol = 2 ** -7 * np.sqrt((rounded.astype(np.float64) ** 2).sum(axis=1, keepdims=True)) * 0.05 + 1e-3
        assert np.all(np.abs(got - ref) <= tol)
        # a head's part alone: its slice of the rows times its slice of the matrix
        h = nh - 1
        ref_h = plain.linear(rounded[:, h * hd:(h + 1) * hd], w.float().cpu().numpy()[:, h * hd:(h + 1) * hd])
        assert np.all(np.abs(parts[h].cpu().numpy() - ref_h) <= tol)


@pytest.mark.parametrize("nh,nkv,hd,K,page,T", [(12, 2, 128, 1536, 16, 64), (4, 2, 64, 1024, 16, 40), (28, 4, 128, 3584, 16, 150),
                                                (6, 2, 32, 768, 8, 130)])
def test_qkv_product_whose_slices_the_rotation_adds(nh, nkv, hd, K, page, T):
    """A q/k/v product whose K the many-rows kernel splits, with the addition of the slices, the bias,
    the rotation and the cache write in one following kernel: the bits of the product with its own
    reduction followed by the rotation kernel."""
    rng = np.random.default_rng(nh + hd + T)
    N = (nh + 2 * nkv) * hd
    x = t32(rng.standard_normal((T, K)).astype(np.float32)).to(torch.bfloat16)
    w = t32((rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)).to(torch.bfloat16)
    b = t32(rng.standard_normal(N).astype(np.float32))
    max_pos = 300
    ang = rng.uniform(0, 6.28, size=(max_pos, hd // 2)).astype(np.float32)
    cos_sin = t32(np.stack([np.cos(ang), np.sin(ang)], axis=-1).astype(np.float32))
    positions = t32(rng.integers(0, max_pos, size=T).astype(np.int32))
    pages = 40
    slots_np = rng.permutation(pages * page)[:T].astype(np.int32)
    slots_np[1] = -1                                   # a row that writes nothing
    slots = t32(slots_np)
    kc = torch.zeros(pages, nkv, page, hd, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    count = ops().qkv_parts_count(x, w, kc, hd, hd)
    assert count > 1, "the shape was meant to be one whose K is split"
    for bias in (b, None):
        kc.zero_(); vc.zero_()
        q = ops().qkv_rope_parts(x, w, bias, positions, cos_sin, slots, kc, vc, nh, nkv, hd, page, count)
        qkv = torch.empty(T, N, dtype=torch.bfloat16, device=DEV)
        ops().gemm_bf16_tc(x, w, bias, qkv)            # the same kernel, its own ordered reduction
        kc2, vc2 = torch.zeros_like(kc), torch.zeros_like(vc)
        ops().rope_kv_write(qkv, positions, cos_sin, slots, kc2, vc2, nh, nkv, hd, hd, page)
        assert torch.equal(q, qkv[:, :nh * hd])
        assert torch.equal(kc, kc2) and torch.equal(vc, vc2)
    ops().check_tc_status(torch.device(DEV))
