"""Each kernel alone against a plain float64 reference of the same operation, at sizes other
than the engine's tiny models use, including ragged ones."""
import math

import numpy as np
import pytest
import torch

from plain import llama_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ops():
    from ithaca_b200.csrc import ops as o
    return o


def close(got, ref, rel):
    got = got.detach().double().cpu()
    ref = ref.detach().double().cpu()
    assert got.shape == ref.shape
    assert torch.isfinite(got).all()
    err = (got - ref).abs().max().item() / max(ref.abs().max().item(), 1e-30)
    assert err <= rel, f"relative error {err:.3e} > {rel:.1e}"


def rnd(shape, seed, dtype=torch.float32, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


# ------------------------------------------------------------------------------------------ simple kernels
@pytest.mark.parametrize("table_dtype", [torch.float32, torch.bfloat16])
def test_embed(table_dtype):
    table = rnd((301, 72), 0, table_dtype)
    ids = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = ops().embed(ids.to(DEV), table.to(DEV), 1.5, status)
    close(out, table.double()[ids.long()] * 1.5, 1e-7)
    assert status.item() == 0
    bad = torch.tensor([3, 301], dtype=torch.int32, device=DEV)
    out = ops().embed(bad, table.to(DEV), 1.0, status)
    assert status.item() == 1 and out[1].abs().max().item() == 0


@pytest.mark.parametrize("d", [64, 200, 202, 4096, 5000, 8192, 8196, 10000])     # rows kept in registers (<= 8192, % 4 == 0) and not
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm(d, out_dtype):
    x = rnd((7, d), 1, scale=3.0)
    w = 1 + rnd((d,), 2, scale=0.1)
    got = ops().rmsnorm(x.to(DEV), w.to(DEV), 1e-5, out_dtype)
    ref = P.rmsnorm(x.double(), w.double(), 1e-5)
    close(got, ref, 2e-6 if out_dtype == torch.float32 else 5e-3)
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    got = ops().rmsnorm(x.to(DEV), w.to(DEV), 1e-5, out_dtype, rows_in=rows)
    close(got, ref[[6, 0, 3]], 2e-6 if out_dtype == torch.float32 else 5e-3)


@pytest.mark.parametrize("ff", [172, 512, 1000])
def test_swiglu(ff):
    gu = rnd((9, 2 * ff), 3, scale=2.0)
    ref = P.silu(gu[:, :ff].double()) * gu[:, ff:].double()
    close(ops().swiglu(gu.to(DEV), torch.float32), ref, 2e-6)
    close(ops().swiglu(gu.to(DEV), torch.bfloat16), ref, 5e-3)


# ------------------------------------------------------------------------------------------ products
@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (5, 172, 64), (33, 70, 172), (130, 257, 300), (64, 384, 192)])
@pytest.mark.parametrize("wdt", [torch.float32, torch.bfloat16])
def test_gemm_simt_float32(M, N, K, wdt):
    x, w = rnd((M, K), 4), rnd((N, K), 5, wdt)
    ref = x.double() @ w.double().T
    got = ops().gemm_simt(x.to(DEV), w.to(DEV))
    close(got, ref, 2e-6)
    base = rnd((M, N), 6)
    got = ops().gemm_simt(x.to(DEV), w.to(DEV), out=base.to(DEV), accumulate=True)
    close(got, ref + base.double(), 2e-6)


def test_gemm_simt_rows_do_not_depend_on_batch():
    """A row's result is the same bits whether it is computed alone or among others."""
    x, w = rnd((37, 300), 7), rnd((129, 300), 8)
    full = ops().gemm_simt(x.to(DEV), w.to(DEV))
    for r in (0, 5, 36):
        one = ops().gemm_simt(x[r:r + 1].to(DEV), w.to(DEV))
        assert torch.equal(one[0], full[r])


@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (8, 200, 72), (9, 4096, 512), (16, 130, 1024), (31, 96, 264),
                                   (64, 300, 2048), (3, 40, 8),
                                   (8, 2048, 8192), (3, 203, 1024), (8, 2368, 1088), (1, 12, 4096)])      # few rows, long K: blocks of 8 rows
@pytest.mark.parametrize("kind", [1, 2])
@pytest.mark.parametrize("ydt", [torch.float32, torch.bfloat16])
def test_gemm_bf16_mma(M, N, K, kind, ydt):
    x, w = rnd((M, K), 9, torch.bfloat16), rnd((N, K), 10, torch.bfloat16)
    ref = x.double() @ w.double().T
    got = ops().gemm_bf16_mma(x.to(DEV), w.to(DEV), out_dtype=ydt, kind=kind)
    assert got is not None
    close(got, ref, 2e-5 if ydt == torch.float32 else 5e-3)
    base = rnd((M, N), 11, ydt)
    got = ops().gemm_bf16_mma(x.to(DEV), w.to(DEV), out=base.to(DEV).clone(), accumulate=True, kind=kind)
    close(got, ref + base.double(), 2e-5 if ydt == torch.float32 else 8e-3)


@pytest.mark.parametrize("M,N,K", [(200, 500, 328), (129, 128, 4096), (1000, 260, 72)])
def test_gemm_bf16_tiled_large(M, N, K):
    x, w = rnd((M, K), 12, torch.bfloat16), rnd((N, K), 13, torch.bfloat16)
    got = ops().gemm_bf16_mma(x.to(DEV), w.to(DEV), kind=2)
    close(got, x.double() @ w.double().T, 2e-5)


@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (8, 200, 72), (17, 4096, 512), (33, 130, 328), (64, 384, 2048),
                                   (100, 96, 264), (200, 500, 1024), (300, 260, 72), (513, 257, 4096)])
@pytest.mark.parametrize("splits", [1, 3, 0])          # whole tiles, K slices, stream-K
@pytest.mark.parametrize("ydt", [torch.float32, torch.bfloat16])
def test_gemm_tcgen05(M, N, K, splits, ydt):
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    x, w = rnd((M, K), 16, torch.bfloat16), rnd((N, K), 17, torch.bfloat16)
    ref = x.double() @ w.double().T
    splits = min(splits, -(-K // 64))
    got = ops().gemm_tcgen05(x.to(DEV), w.to(DEV), out_dtype=ydt, splits=splits, status=status)
    assert got is not None and status.item() == 0
    close(got, ref, 2e-5 if ydt == torch.float32 else 5e-3)
    base = rnd((M, N), 18, ydt)
    got = ops().gemm_tcgen05(x.to(DEV), w.to(DEV), out=base.to(DEV).clone(), accumulate=True, splits=splits, status=status)
    assert status.item() == 0
    close(got, ref + base.double(), 2e-5 if ydt == torch.float32 else 8e-3)


@pytest.mark.parametrize("M,N,K,n_cl", [(17, 4096, 512, 2), (17, 4096, 512, 4), (64, 384, 2048, 3), (33, 130, 328, 3),
                                        (100, 96, 264, 2), (128, 4096, 1024, 2), (1, 200, 4096, 4), (64, 6000, 4096, 3)])
@pytest.mark.parametrize("ydt", [torch.float32, torch.bfloat16])
def test_gemm_tcgen05_cluster_mode(M, N, K, n_cl, ydt):
    """Few tiles: clusters of 2 to 4 blocks share a tile, each a slice of K, and the block of rank 0 adds the
    others' sums from its shared memory in rank order.  Plain, accumulating, the same bits every time; and the
    shapes the mode does not take are refused, not computed."""
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert ops().tcgen05_cluster_fits(M, N, K, n_cl)
    x, w = rnd((M, K), 26, torch.bfloat16).to(DEV), rnd((N, K), 27, torch.bfloat16).to(DEV)
    ref = x.double().cpu() @ w.double().cpu().T
    got = ops().gemm_tcgen05(x, w, out_dtype=ydt, splits=-n_cl, status=status)
    assert got is not None and status.item() == 0
    close(got, ref, 2e-5 if ydt == torch.float32 else 5e-3)
    for _ in range(3):
        assert torch.equal(ops().gemm_tcgen05(x, w, out_dtype=ydt, splits=-n_cl, status=status), got)
    base = rnd((M, N), 28, ydt)
    acc = ops().gemm_tcgen05(x, w, out=base.to(DEV).clone(), accumulate=True, splits=-n_cl, status=status)
    close(acc, ref + base.double(), 2e-5 if ydt == torch.float32 else 8e-3)
    assert status.item() == 0


def test_gemm_tcgen05_cluster_mode_refuses_what_it_does_not_take():
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for M, N, K, n_cl in [(300, 256, 512, 2), (100, 256, 512, 3), (17, 128 * 80, 512, 2), (17, 256, 64, 2), (17, 256, 512, 5)]:
        assert not ops().tcgen05_cluster_fits(M, N, K, n_cl)
        x, w = rnd((M, K), 1, torch.bfloat16).to(DEV), rnd((N, K), 2, torch.bfloat16).to(DEV)
        out = torch.full((M, N), 3.0, device=DEV)
        assert ops().gemm_tcgen05(x, w, out=out, splits=-n_cl, status=status) is None
        assert float(out.min()) == 3.0 and float(out.max()) == 3.0
    assert status.item() == 0


@pytest.mark.parametrize("M,N,K", [(300, 260, 72), (513, 257, 4096), (2048, 4096, 512), (1000, 128, 264), (700, 1300, 1024)])
@pytest.mark.parametrize("ydt", [torch.float32, torch.bfloat16])
def test_gemm_tcgen05_pair_mode(M, N, K, ydt):
    """More than 256 tokens: pairs of blocks take two weight tiles each and share one copy of every token tile (half
    of its rows fetched by each block into both).  Odd numbers of weight tiles leave a block of the last pair with
    a tile that does not exist.  The sums run in the same order as without pairs, so the results are the same bits."""
    if ops().pairs_lib() is None:
        pytest.skip("the pair mode's library is not part of this checkout")
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    x, w = rnd((M, K), 36, torch.bfloat16).to(DEV), rnd((N, K), 37, torch.bfloat16).to(DEV)
    ref = x.double().cpu() @ w.double().cpu().T
    got = ops().gemm_tcgen05(x, w, out_dtype=ydt, splits=1, status=status, pairs=True)
    assert got is not None and status.item() == 0
    close(got, ref, 2e-5 if ydt == torch.float32 else 5e-3)
    plain = ops().gemm_tcgen05(x, w, out_dtype=ydt, splits=1, status=status, pairs=False)
    assert torch.equal(got, plain)
    base = rnd((M, N), 38, ydt).to(DEV)
    acc = ops().gemm_tcgen05(x, w, out=base.clone(), accumulate=True, splits=1, status=status, pairs=True)
    assert torch.equal(acc, ops().gemm_tcgen05(x, w, out=base.clone(), accumulate=True, splits=1, status=status, pairs=False))
    for _ in range(3):                                       # back to back: stages and barriers of both blocks stay in step
        assert torch.equal(ops().gemm_tcgen05(x, w, out_dtype=ydt, splits=1, status=status, pairs=True), got)
    assert status.item() == 0


def test_tcgen05_issue_rate_measurement():
    """The measurement of what issuing costs runs, ends within its bounded waits, and shows the two facts the product's
    modes rest on: a 256-wide product instruction keeps the tensor core busy for about 128 cycles, and narrow ones are
    bound by the issuing thread, so that two threads issue them about twice as fast."""
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    wide = ops().tcgen05_issue_rate(256, 8, 1, status)
    narrow = ops().tcgen05_issue_rate(64, 8, 1, status)
    narrow2 = ops().tcgen05_issue_rate(64, 8, 2, status)
    assert status.item() == 0
    assert 120 <= wide <= 160, wide
    assert 40 <= narrow <= wide, narrow
    assert narrow2 / 2 < 0.7 * narrow, (narrow, narrow2)


def test_gemm_tcgen05_stream_k_back_to_back():
    """Stream-K products of different shapes one after another share one scratch: every launch leaves the
    flags as it found them, a tile cut into many pieces (one tile, K = 8192) sums them in K order, and the
    result is the same bits every time."""
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    cases = [(129, 128, 8192), (64, 384, 2048), (40, 1000, 520), (129, 128, 8192), (300, 4096, 1024)]
    data = [(rnd((M, K), 30 + i, torch.bfloat16).to(DEV), rnd((N, K), 40 + i, torch.bfloat16).to(DEV)) for i, (M, N, K) in enumerate(cases)]
    first = {}
    for rep in range(3):
        for i, (x, w) in enumerate(data):
            got = ops().gemm_tcgen05(x, w, splits=0, status=status)
            if rep == 0:
                close(got, x.double().cpu() @ w.double().cpu().T, 2e-5)
                first[i] = got.clone()
            else:
                assert torch.equal(got, first[i])
    assert status.item() == 0
    flags = ops().stream_k_scratch(DEV)[:4096].view(torch.int32)      # the scratch begins with the flags
    assert int(flags.abs().max().item()) == 0


def test_gemm_tcgen05_strided_rows_and_default_splits():
    """Rows that are slices of wider matrices (row stride > K), and the split the dispatcher picks."""
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    xb, wb = rnd((40, 640), 19, torch.bfloat16).to(DEV), rnd((4096, 1024), 20, torch.bfloat16).to(DEV)
    x, w = xb[:, 128:640], wb[:, 512:1024]
    out = torch.zeros((40, 8192), device=DEV)
    got = ops().gemm_tcgen05(x, w, out=out[:, 4096:], status=status)
    assert got is not None and status.item() == 0 and ops().tcgen05_splits(40, 4096, 512) == 2      # K slices
    assert ops().tcgen05_splits(40, 28672, 4096) == 0 and ops().tcgen05_splits(2048, 28672, 4096) == 1   # stream-K; whole tiles
    close(out[:, 4096:], x.double() @ w.double().T, 2e-5)
    assert out[:, :4096].abs().max().item() == 0
    assert ops().gemm_tcgen05(xb[:, 4:516], wb[:, :512], status=status) is None          # rows not 16-byte aligned


@pytest.mark.parametrize("M", [1, 8, 13, 16, 17, 64, 300])
@pytest.mark.parametrize("ff,d", [(172, 64), (512, 192), (1000, 264), (4096, 1024), (600, 1024)])
def test_gate_up_product_with_swiglu_epilogue(M, ff, d):
    """h = silu(x Wg^T) * (x Wu^T) from one kernel over row-interleaved weights, every dispatch path."""
    from ithaca_b200.csrc import gemm_bf16
    x = rnd((M, d), 21, torch.bfloat16)
    wg, wu = rnd((ff, d), 22, torch.bfloat16, 0.3), rnd((ff, d), 23, torch.bfloat16, 0.3)
    ref = P.silu(x.double() @ wg.double().T) * (x.double() @ wu.double().T)
    wi = torch.stack((wg, wu), dim=1).reshape(2 * ff, d).contiguous().to(DEV)
    got = gemm_bf16.gemm_swiglu(x.to(DEV), wi)
    assert got.dtype == torch.bfloat16 and got.shape == (M, ff)
    close(got, ref, 6e-3)
    status = ops().device_status(DEV)
    if M > 8:                                            # 9-16 tokens go to either kernel, by the matrix's size
        for splits in (1, 3, 0, -2):
            if splits < 0 and not ops().tcgen05_cluster_fits(M, 2 * ff, d, -splits):
                continue
            got = ops().gemm_tcgen05(x.to(DEV), wi, out_dtype=torch.float32, splits=min(splits, -(-d // 64)), status=status,
                                     swiglu=True)
            close(got, ref, 2e-5)
    if M <= 16:
        close(ops().gemm_bf16_mma(x.to(DEV), wi, out_dtype=torch.float32, kind=1, swiglu=True), ref, 2e-5)
    assert status.item() == 0


def test_swiglu_kernel_interleaved():
    gu = rnd((5, 2 * 172), 24, scale=2.0)
    ref = P.silu(gu[:, 0::2].double()) * gu[:, 1::2].double()
    close(ops().swiglu(gu.to(DEV), torch.float32, interleaved=True), ref, 2e-6)


def test_gemm_bf16_refuses_unaligned_k():
    x, w = rnd((4, 172), 14, torch.bfloat16), rnd((64, 172), 15, torch.bfloat16)
    assert ops().gemm_bf16_mma(x.to(DEV), w.to(DEV)) is None           # K % 8 != 0
    from ithaca_b200.csrc import gemm_bf16
    close(gemm_bf16.gemm(x.to(DEV), w.to(DEV)), x.double() @ w.double().T, 2e-5)   # the dispatcher falls back


# ------------------------------------------------------------------------------------------ rotary + cache
class Paged:
    """Sequences laid into pages in a scrambled order, the way a used cache looks."""

    def __init__(self, lens, nkv, hd, dtype, seed, page=64, spare=3):
        self.page, self.nkv, self.hd = page, nkv, hd
        need = sum(-(-l // page) for l in lens)
        self.n_pages = need + spare
        perm = np.random.default_rng(seed).permutation(self.n_pages)[:need]
        cols = max(-(-l // page) for l in lens)
        self.table = np.full((len(lens), cols), -1, dtype=np.int32)
        it = iter(perm)
        for b, l in enumerate(lens):
            for c in range(-(-l // page)):
                self.table[b, c] = next(it)
        self.k = torch.zeros((self.n_pages, nkv, page, hd), dtype=dtype)
        self.v = torch.zeros_like(self.k)
        self.lens = list(lens)

    def fill(self, ks, vs):
        for b, (k, v) in enumerate(zip(ks, vs)):
            for j in range(k.shape[0]):
                pg = self.table[b, j // self.page]
                self.k[pg, :, j % self.page] = k[j].to(self.k.dtype)
                self.v[pg, :, j % self.page] = v[j].to(self.v.dtype)

    def dev(self):
        return self.k.to(DEV), self.v.to(DEV), torch.from_numpy(self.table).to(DEV)


@pytest.mark.parametrize("nh,nkv,hd,rot,pairing", [(4, 4, 16, 16, 0), (6, 2, 32, 32, 1), (5, 1, 48, 32, 0)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rope_append(nh, nkv, hd, rot, pairing, dtype):
    lens, new = [70, 5, 130], [3, 5, 66]                    # sequence lengths after the step, tokens it brings
    T = sum(new)
    qkv = rnd((T, (nh + 2 * nkv) * hd), 20)
    inv = P.rope_inv_freq(rot, 10000.0, None)
    pg = Paged(lens, nkv, hd, dtype, seed=1)
    token_seq = np.repeat(np.arange(3), new).astype(np.int32)
    token_pos = np.concatenate([np.arange(l - n, l) for l, n in zip(lens, new)]).astype(np.int32)
    k_d, v_d, tab = pg.dev()
    q_out = torch.empty((T, nh * hd), dtype=dtype, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops().rope_append(qkv.to(DEV), q_out, k_d, v_d, torch.from_numpy(token_seq).to(DEV),
                      torch.from_numpy(token_pos).to(DEV), tab, inv.to(DEV), nh, nkv, hd, rot, pairing, True, status)
    assert status.item() == 0
    x = qkv.double().view(T, nh + 2 * nkv, hd)
    pos = torch.from_numpy(token_pos)
    name = "half" if pairing == 0 else "interleaved"
    q_ref = P.rope(x[:, :nh], pos, inv, name)
    k_ref = P.rope(x[:, nh:nh + nkv], pos, inv, name)
    v_ref = x[:, nh + nkv:]
    tol = 2e-6 if dtype == torch.float32 else 5e-3
    close(q_out.view(T, nh, hd), q_ref, tol)
    k_h, v_h = k_d.cpu(), v_d.cpu()
    got_k = torch.stack([k_h[pg.table[s, p // 64], :, p % 64] for s, p in zip(token_seq, token_pos)])
    got_v = torch.stack([v_h[pg.table[s, p // 64], :, p % 64] for s, p in zip(token_seq, token_pos)])
    close(got_k, k_ref, tol)
    close(got_v, v_ref, tol)
    # nothing else in the pool was touched
    touched = torch.zeros(k_h.shape[0], 64, dtype=torch.bool)
    for s, p in zip(token_seq, token_pos):
        touched[pg.table[s, p // 64], p % 64] = True
    assert k_h.float().abs().sum(dim=(1, 3))[~touched].max().item() == 0


@pytest.mark.parametrize("nh,nkv,hd,d", [(4, 4, 16, 264), (6, 2, 32, 264), (5, 1, 48, 264), (8, 2, 128, 264),
                                         (6, 2, 32, 1024)])      # the last: few rows and a long K, the skinny kernel's blocks of 8 rows
@pytest.mark.parametrize("T_new", [[3, 5, 1], [20, 7, 30], [40, 30, 66], [300, 2, 70]])
def test_qkv_product_with_rotary_and_cache_epilogue(nh, nkv, hd, d, T_new):
    """x W^T, rotated, with q to its buffer and k, v into the pages, from one kernel: every dispatch path
    (skinny, tcgen05 with whole tiles and stream-K) against the plain product followed by the plain rotation."""
    new = T_new
    lens = [n + e for n, e in zip(new, (70, 0, 64))]
    T = sum(new)
    x = rnd((T, d), 50, torch.bfloat16)
    wq, wk, wv = rnd((nh * hd, d), 51, torch.bfloat16, 0.2), rnd((nkv * hd, d), 52, torch.bfloat16, 0.2), rnd((nkv * hd, d), 53, torch.bfloat16, 0.2)
    inv = P.rope_inv_freq(hd, 10000.0, None)
    token_seq = np.repeat(np.arange(3), new).astype(np.int32)
    token_pos = np.concatenate([np.arange(l - n, l) for l, n in zip(lens, new)]).astype(np.int32)
    pos = torch.from_numpy(token_pos)
    q_ref = P.rope((x.double() @ wq.double().T).view(T, nh, hd), pos, inv, "half")
    k_ref = P.rope((x.double() @ wk.double().T).view(T, nkv, hd), pos, inv, "half")
    v_ref = (x.double() @ wv.double().T).view(T, nkv, hd)
    half = hd // 2
    order = torch.stack((torch.arange(half), torch.arange(half) + half), dim=1).reshape(-1)     # (i, i+half) -> (2i, 2i+1)
    w = torch.cat((wq.view(nh, hd, d)[:, order].reshape(nh * hd, d), wk.view(nkv, hd, d)[:, order].reshape(nkv * hd, d), wv)).to(DEV)
    pg = Paged(lens, nkv, hd, torch.bfloat16, seed=3)
    k_d, v_d, tab = pg.dev()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    cs = ops().rope_table(pos.to(DEV), inv.to(DEV))
    ang = pos.float()[:, None] * inv[None, :]
    close(cs[..., 0], torch.cos(ang.double()), 2e-6)
    close(cs[..., 1], torch.sin(ang.double()), 2e-6)
    q_out = torch.zeros((T, nh * hd), dtype=torch.bfloat16, device=DEV)
    ok = ops().gemm_qkv_rope(x.to(DEV), w, q_out, k_d, v_d, cs, torch.from_numpy(token_seq).to(DEV), pos.to(DEV), tab,
                             nh, nkv, hd, True, status)
    assert ok and status.item() == 0
    close(q_out.view(T, nh, hd), q_ref[:, :, order], 6e-3)
    k_h, v_h = k_d.cpu(), v_d.cpu()
    got_k = torch.stack([k_h[pg.table[s, p // 64], :, p % 64] for s, p in zip(token_seq, token_pos)])
    got_v = torch.stack([v_h[pg.table[s, p // 64], :, p % 64] for s, p in zip(token_seq, token_pos)])
    close(got_k, k_ref[:, :, order], 6e-3)
    close(got_v, v_ref, 6e-3)
    touched = torch.zeros(k_h.shape[0], 64, dtype=torch.bool)
    for s, p in zip(token_seq, token_pos):
        touched[pg.table[s, p // 64], p % 64] = True
    assert k_h.float().abs().sum(dim=(1, 3))[~touched].max().item() == 0 and v_h.float().abs().sum(dim=(1, 3))[~touched].max().item() == 0
    # the cluster mode of the tcgen05 product through the same epilogue
    N_all = (nh + 2 * nkv) * hd
    if T > 16 and ops().tcgen05_cluster_fits(T, N_all, d, 2):
        q3, (k3, v3, _) = torch.zeros_like(q_out), pg.dev()
        assert ops().gemm_qkv_rope(x.to(DEV), w, q3, k3, v3, cs, torch.from_numpy(token_seq).to(DEV), pos.to(DEV), tab,
                                   nh, nkv, hd, True, status, splits=-2)
        close(q3.view(T, nh, hd), q_ref[:, :, order], 6e-3)
        k3h = k3.cpu()
        close(torch.stack([k3h[pg.table[s, p // 64], :, p % 64] for s, p in zip(token_seq, token_pos)]), k_ref[:, :, order], 6e-3)
        assert status.item() == 0
    # whole tiles, which more than 256 tokens run in the pair mode where its library is there
    if T > 256:
        q4, (k4, v4, _) = torch.zeros_like(q_out), pg.dev()
        assert ops().gemm_qkv_rope(x.to(DEV), w, q4, k4, v4, cs, torch.from_numpy(token_seq).to(DEV), pos.to(DEV), tab,
                                   nh, nkv, hd, True, status, splits=1)
        close(q4.view(T, nh, hd), q_ref[:, :, order], 6e-3)
        k4h, v4h = k4.cpu(), v4.cpu()
        close(torch.stack([k4h[pg.table[s, p // 64], :, p % 64] for s, p in zip(token_seq, token_pos)]), k_ref[:, :, order], 6e-3)
        close(torch.stack([v4h[pg.table[s, p // 64], :, p % 64] for s, p in zip(token_seq, token_pos)]), v_ref, 6e-3)
        assert status.item() == 0
    # without the right to write the cache only q appears
    k2, v2 = torch.zeros_like(k_d), torch.zeros_like(v_d)
    assert ops().gemm_qkv_rope(x.to(DEV), w, q_out, k2, v2, cs, torch.from_numpy(token_seq).to(DEV), pos.to(DEV), tab,
                               nh, nkv, hd, False, status)
    assert k2.abs().max().item() == 0 and v2.abs().max().item() == 0


# ------------------------------------------------------------------------------------------ attention
def attention_case(nh, nkv, hd, lens, new, window, dtype, seed, boost=None):
    """Random q/k/v for sequences of the given lengths, the last ``new[b]`` tokens of each being
    this step's queries.  Returns everything the kernels need plus the plain result."""
    g = torch.Generator().manual_seed(seed)
    ks = [torch.randn((l, nkv, hd), generator=g) for l in lens]
    vs = [torch.randn((l, nkv, hd), generator=g) for l in lens]
    qs = [torch.randn((l, nh, hd), generator=g) for l in lens]
    if boost is not None:
        boost(qs, ks, vs)
    ks = [k.to(dtype) for k in ks]
    vs = [v.to(dtype) for v in vs]
    qs = [q.to(dtype) for q in qs]
    pg = Paged(lens, nkv, hd, dtype, seed)
    pg.fill(ks, vs)
    ref = torch.cat([P.attention(q.double(), k.double(), v.double(), window=window)[l - n:]
                     for q, k, v, l, n in zip(qs, ks, vs, lens, new)])
    q_step = torch.cat([q[l - n:] for q, l, n in zip(qs, lens, new)]).reshape(sum(new), nh * hd)
    token_seq = np.repeat(np.arange(len(lens)), new).astype(np.int32)
    token_pos = np.concatenate([np.arange(l - n, l) for l, n in zip(lens, new)]).astype(np.int32)
    cu = np.concatenate([[0], np.cumsum(new)]).astype(np.int32)
    return dict(q=q_step.to(DEV), pg=pg, ref=ref.reshape(sum(new), nh * hd), token_seq=torch.from_numpy(token_seq).to(DEV),
                token_pos=torch.from_numpy(token_pos).to(DEV), cu=torch.from_numpy(cu).to(DEV),
                kv_lens=torch.tensor(lens, dtype=torch.int32, device=DEV))


SHAPES = [(4, 4, 16), (6, 2, 32), (5, 1, 48), (8, 2, 64), (8, 4, 128)]


@pytest.mark.parametrize("nh,nkv,hd", SHAPES)
@pytest.mark.parametrize("window", [0, 40])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_simt(nh, nkv, hd, window, dtype):
    lens, new = [1, 70, 200, 129], [1, 70, 3, 1]
    c = attention_case(nh, nkv, hd, lens, new, window or None, dtype, seed=30)
    k_d, v_d, tab = c["pg"].dev()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    got = ops().attention_simt(c["q"], k_d, v_d, c["token_seq"], c["token_pos"], tab, nh, 1 / math.sqrt(hd), window,
                               status)
    assert status.item() == 0
    close(got, c["ref"], 3e-6 if dtype == torch.float32 else 8e-3)


@pytest.mark.parametrize("nh,nkv,hd,kind", [s + ("mma",) for s in SHAPES] + [(8, 2, 64, "tc"), (8, 4, 128, "tc"),
                                                                            (4, 4, 128, "tc")])
@pytest.mark.parametrize("window", [0, 40, 100])
def test_attention_bf16_prefill(nh, nkv, hd, kind, window):
    from ithaca_b200.csrc import attention_bf16 as A
    lens, new = [1, 70, 200, 129, 64, 700], [1, 70, 67, 129, 5, 450]       # whole prompts and later chunks
    c = attention_case(nh, nkv, hd, lens, new, window or None, torch.bfloat16, seed=31)
    k_d, v_d, tab = c["pg"].dev()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    got = A.prefill(c["q"], k_d, v_d, c["cu"], c["kv_lens"], tab, len(lens), max(new), nh, 1 / math.sqrt(hd), window,
                    status, kind=kind)
    assert status.item() == 0
    close(got, c["ref"], 8e-3)


@pytest.mark.parametrize("hd,window", [(128, 40), (128, 8), (64, 40), (128, 0)])
def test_attention_tcgen05_many_tiles_of_few_pages(hd, window):
    """Hundreds of blocks that each see two to four pages (a narrow window), several per SM at a time: what one
    block's roles hand to each other (rings, score buffers, the last product before the output is read) is
    exercised at every block's start and end rather than in a long steady state.  Run a few times: a missing
    wait shows only when the timing falls that way."""
    from ithaca_b200.csrc import attention_bf16 as A
    nh, nkv = 20, 5
    lens, new = [1300, 2000, 130], [1300, 900, 130]
    c = attention_case(nh, nkv, hd, lens, new, window or None, torch.bfloat16, seed=33)
    k_d, v_d, tab = c["pg"].dev()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for _ in range(4):
        got = A.prefill(c["q"], k_d, v_d, c["cu"], c["kv_lens"], tab, len(lens), max(new), nh, 1 / math.sqrt(hd), window,
                        status, kind="tc")
        assert status.item() == 0
        close(got, c["ref"], 8e-3)


@pytest.mark.parametrize("hd", [64, 128])
def test_attention_tcgen05_thousands_of_two_page_tiles(hd):
    """Tiles that see exactly two pages, thousands of blocks, many times over.  With two products per tile the wait for
    the last one once named its phase on a barrier that could by then stand two phases on; it showed on one box
    only, a few times in ten thousand blocks.  Every run must give the first run's bits and leave the status word clean."""
    from ithaca_b200.csrc import attention_bf16 as A
    nh, nkv = 16, 4
    lens = [128] * 48 + [100] * 32 + [65] * 16
    c = attention_case(nh, nkv, hd, lens, lens, None, torch.bfloat16, seed=35)
    k_d, v_d, tab = c["pg"].dev()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    first = None
    for rep in range(60):
        got = A.prefill(c["q"], k_d, v_d, c["cu"], c["kv_lens"], tab, len(lens), max(lens), nh, 1 / math.sqrt(hd), 0,
                        status, kind="tc")
        if first is None:
            first = got.clone()
            close(got, c["ref"], 8e-3)
        else:
            assert torch.equal(got, first), rep
    assert status.item() == 0


@pytest.mark.parametrize("nh,nkv,hd", SHAPES)
@pytest.mark.parametrize("window", [0, 40, 300])
def test_attention_bf16_decode(nh, nkv, hd, window):
    from ithaca_b200.csrc import attention_bf16 as A
    lens = [1, 64, 65, 257, 700, 1030]
    new = [1] * len(lens)
    c = attention_case(nh, nkv, hd, lens, new, window or None, torch.bfloat16, seed=32)
    k_d, v_d, tab = c["pg"].dev()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for bound, chunk in ((max(lens), 4), (2048, 4), (max(lens), 2), (2048, 16)):   # a larger grid or other chunks change nothing
        got = A.decode(c["q"], k_d, v_d, c["kv_lens"], tab, len(lens), bound, nh, 1 / math.sqrt(hd), window, status,
                       chunk_pages=chunk)
        assert status.item() == 0
        close(got, c["ref"], 8e-3)


@pytest.mark.parametrize("kind", ["simt32", "prefill", "prefill_tc", "decode"])
def test_attention_reaches_a_far_key_and_respects_the_window_edge(kind):
    """One key far back is made to dominate the last query's scores: the output must be that
    key's value.  Under a window the same key just outside must not count, just inside must."""
    from ithaca_b200.csrc import attention_bf16 as A
    nh, nkv, hd, L = 4, 2, 64, 700
    dtype = torch.float32 if kind == "simt32" else torch.bfloat16
    for window, far in [(0, 3), (0, 130), (100, L - 100), (100, L - 101)]:
        def boost(qs, ks, vs, far=far):
            d = torch.zeros(hd)
            d[0] = 1.0
            qs[0][L - 1] = d * 40.0
            ks[0][:] *= 0.05
            ks[0][far] = d * 40.0
        n_new = 1 if kind == "decode" else 5
        c = attention_case(nh, nkv, hd, [L], [n_new], window or None, dtype, seed=33, boost=boost)
        k_d, v_d, tab = c["pg"].dev()
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        scale = 1 / math.sqrt(hd)
        if kind == "simt32":
            got = ops().attention_simt(c["q"], k_d, v_d, c["token_seq"], c["token_pos"], tab, nh, scale, window, status)
        elif kind in ("prefill", "prefill_tc"):
            got = A.prefill(c["q"], k_d, v_d, c["cu"], c["kv_lens"], tab, 1, n_new, nh, scale, window, status,
                            kind="mma" if kind == "prefill" else "tc")
        else:
            got = A.decode(c["q"], k_d, v_d, c["kv_lens"], tab, 1, L, nh, scale, window, status)
        close(got, c["ref"], 3e-6 if dtype == torch.float32 else 8e-3)
        # the construction does what it says: inside the reach the far value is the output
        pgt = c["pg"]
        far_v = pgt.v[pgt.table[0, far // 64], :, far % 64].double()          # [nkv, hd]
        last = got[-1].double().cpu().view(nh, hd)
        inside = window == 0 or far > L - 1 - window
        hit = (last - far_v.repeat_interleave(nh // nkv, 0)).abs().max().item() < 0.05
        assert hit == inside


# ------------------------------------------------------------------------------------------ sampling
@pytest.mark.parametrize("V", [3001, 16384, 50021])        # one block a row; rows cut into slices (vocabulary >= 16 Ki)
def test_argmax_takes_the_first_of_equal_maxima(V):
    lg = rnd((5, V), 40)
    lg[2, 77] = lg[2, V - 501] = 9.0                         # equal maxima in different slices: the lower index wins
    lg[4, V - 1] = 11.0                                      # the very last entry
    want = [int(torch.argmax(r)) for r in lg[:2]] + [77, int(torch.argmax(lg[3])), V - 1]
    for _ in range(3):                                       # the slices' counters are left clear for the next call
        assert ops().argmax(lg.to(DEV)).cpu().tolist() == want
    wide = torch.zeros((5, V + 13))                          # rows that are slices of wider rows
    wide[:, :V] = lg
    assert ops().argmax(wide.to(DEV)[:, :V]).cpu().tolist() == want


@pytest.mark.parametrize("V", [256, 384, 5003])
@pytest.mark.parametrize("temp,top_k,top_p,pen", [(0.8, 40, 0.9, 1.1), (1.0, 5, 1.0, 1.0), (0.7, 100000, 0.5, 1.3),
                                                  (1.5, 1, 0.9, 1.0), (0.0, 40, 0.9, 1.2), (2.0, 100000, 1.0, 1.0)])
def test_sample_matches_plain(V, temp, top_k, top_p, pen):
    rows = 12
    lg = rnd((rows, V), 41, scale=2.0)
    lg[3, 10] = lg[3, 200] = lg[3].max() + 0.5                                  # equal maxima
    recent = [[(7 * r + i * i) % V for i in range(r % 5 + (r > 6) * 60)] for r in range(rows)]
    rec = torch.full((rows, 64), -1, dtype=torch.int32)
    for r, ids in enumerate(recent):
        ids = ids[-64:]
        rec[r, :len(ids)] = torch.tensor(ids, dtype=torch.int32)
    streams = torch.arange(rows, dtype=torch.int32) * 3
    for counter in (0, 1, 17):
        counters = torch.full((rows,), counter, dtype=torch.int32)
        got = ops().sample(lg.to(DEV), temp, top_k, top_p, pen, rec.to(DEV), 1234, streams.to(DEV),
                           counters.to(DEV)).cpu().tolist()
        want = [P.sample(lg[r], temp, top_k, top_p, pen, recent[r][-64:], P.philox_uniform(1234, int(streams[r]), counter))
                for r in range(rows)]
        assert got == want


@pytest.mark.parametrize("V", [50021, 128256])
@pytest.mark.parametrize("shape", ["random", "ties", "flat", "peaked"])
@pytest.mark.parametrize("temp,top_k,top_p,pen", [(0.8, 40, 0.9, 1.1), (1.0, 1000, 0.95, 1.3), (1.2, 3000, 0.8, 1.0)])
def test_sample_at_large_vocabularies(V, shape, temp, top_k, top_p, pen):
    """The kernel's short cuts for few kept candidates (a bound from the threads' own maxima; the k-th largest by
    digits when too many lie above it) and the general path (more than 1,024 kept), on rows that look like
    logits, on rows of few distinct values (thousands of equal entries at the cut), on a constant row and on a
    row with one entry far above the rest."""
    rows = 4
    lg = rnd((rows, V), 43, scale=2.0)
    if shape == "ties":
        lg = (lg * 2).round() / 2
    elif shape == "flat":
        lg = torch.zeros_like(lg) + 0.25
        lg[1, 77] = 0.5
    elif shape == "peaked":
        lg[:, 4321] += 30.0
    recent = [[(7 * r + i * i) % V for i in range(r * 9)] for r in range(rows)]
    rec = torch.full((rows, 64), -1, dtype=torch.int32)
    for r, ids in enumerate(recent):
        rec[r, :len(ids)] = torch.tensor(ids, dtype=torch.int32)
    streams = torch.arange(rows, dtype=torch.int32) + 5
    for counter in (3,):
        counters = torch.full((rows,), counter, dtype=torch.int32)
        got = ops().sample(lg.to(DEV), temp, top_k, top_p, pen, rec.to(DEV), 77, streams.to(DEV), counters.to(DEV)).cpu().tolist()
        want = [P.sample(lg[r], temp, top_k, top_p, pen, recent[r], P.philox_uniform(77, int(streams[r]), counter))
                for r in range(rows)]
        assert got == want


def test_sample_follows_the_distribution():
    """Many draws from one row: frequencies follow exp(l / temp) over the kept candidates."""
    V, n = 50, 4000
    lg = rnd((1, V), 42, scale=1.5).repeat(n, 1).contiguous()
    got = ops().sample(lg.to(DEV), 1.0, 8, 1.0, 1.0, None, 99, torch.zeros(n, dtype=torch.int32, device=DEV),
                       torch.arange(n, dtype=torch.int32, device=DEV)).cpu()
    top = torch.topk(lg[0], 8).indices
    assert set(got.tolist()) <= set(top.tolist())
    p = torch.softmax(lg[0][top].double(), 0)
    freq = torch.tensor([(got == i).sum().item() for i in top], dtype=torch.double) / n
    assert (freq - p).abs().max().item() < 4 * math.sqrt(0.25 / n)


def test_a_wait_that_nothing_satisfies_gives_up_and_returns():
    """The tensor-core kernels wait on barriers and flags with a limit.  Here the limit is 1 ms and nothing ever
    arrives: the wait returns false after about that long, the event is recorded in the status word (bit of
    code 4), the block's abort flag is up, a second waiter of the block leaves at once although its own limit is
    far away, the wait on a global flag runs out the same way, and the device goes on working afterwards."""
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    res = ops().selftest_wait_expires(status, limit_ns=1_000_000).cpu().tolist()
    assert res[0] == 0 and res[1] == 1, res                  # gave up; abort flag raised
    assert 900 <= res[2] <= 20000, res                       # after about a millisecond
    assert res[3] == 0 and res[4] < 500, res                 # the second waiter saw the flag, not its 200 ms
    assert res[5] == 0, res                                  # the flag wait of the stream-K pieces, too
    assert status.item() == 1 << 3
    # a product given that status word returns at once and leaves its output alone; with a clean word it computes
    x, w = rnd((40, 256), 1, torch.bfloat16).to(DEV), rnd((256, 256), 2, torch.bfloat16).to(DEV)
    out = torch.full((40, 256), 7.0, device=DEV)
    ops().gemm_tcgen05(x, w, out=out, status=status, splits=1)
    assert float(out.min()) == 7.0 and float(out.max()) == 7.0
    status.zero_()
    ops().gemm_tcgen05(x, w, out=out, status=status, splits=1)
    close(out, x.double().cpu() @ w.double().cpu().T, 2e-5)
    assert status.item() == 0
