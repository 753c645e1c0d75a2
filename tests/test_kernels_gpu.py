"""Each CUDA kernel alone against plain PyTorch float32 math, at sizes other than the engine's
(odd widths, head sizes in steps of 16, group sizes 1..5, vocabularies that are no power of two)."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, scale=1.0):
    return dict(atol=(2e-5 if dtype == torch.float32 else 1.6e-2) * scale, rtol=1e-5 if dtype == torch.float32 else 1.6e-2)


@pytest.fixture(scope="module")
def ops():
    from tandem_b200.kernels import ops as o

    return o


def dev(t):
    return t.to("cuda")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H,V", [(1, 64, 50), (7, 100, 1000), (33, 4096, 777)])
def test_embedding(ops, dtype, T, H, V):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(V, H, generator=g).to(dtype)
    ids = torch.randint(0, V, (T,), generator=g, dtype=torch.int32)
    out = ops.embedding(dev(ids), dev(table))
    assert out.dtype == torch.float32
    torch.testing.assert_close(out.cpu(), table[ids.long()].float(), atol=0, rtol=0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H,eps", [(1, 64, 1e-6), (5, 100, 1e-5), (19, 4096, 1e-6), (3, 5120, 3e-6), (2, 7, 1e-2),
                                     (513, 4096, 1e-6), (600, 1000, 1e-5), (1025, 104, 1e-6)])
def test_add_rmsnorm(ops, dtype, T, H, eps):
    g = torch.Generator().manual_seed(1)
    x = torch.randn(T, H, generator=g).to(dtype)
    res = torch.randn(T, H, generator=g) * 3
    w = 1 + 0.1 * torch.randn(H, generator=g)
    s = x.float() + res
    want = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + eps) * w
    res_d = dev(res.clone())
    y = ops.add_rmsnorm(dev(x), res_d, dev(w), eps, dtype)
    torch.testing.assert_close(res_d.cpu(), s, atol=1e-6, rtol=1e-6)  # the residual sum is float32
    torch.testing.assert_close(y.cpu().float(), want, **tol(dtype))
    # without x: plain norm, the residual untouched; with rows: only those rows, in that order
    res_d = dev(res.clone())
    y = ops.add_rmsnorm(None, res_d, dev(w), eps, dtype)
    torch.testing.assert_close(res_d.cpu(), res, atol=0, rtol=0)
    torch.testing.assert_close(y.cpu().float(), res * torch.rsqrt(res.pow(2).mean(-1, keepdim=True) + eps) * w, **tol(dtype))
    rows = torch.tensor([T - 1, 0], dtype=torch.int32)[: min(2, T)]
    res_d = dev(res.clone())
    y = ops.add_rmsnorm(dev(x), res_d, dev(w), eps, dtype, rows=dev(rows))
    torch.testing.assert_close(y.cpu().float(), want[rows.long()], **tol(dtype))


def _rope_reference(x, pos, theta, rd):
    half = rd // 2
    inv = 1.0 / (theta ** (torch.arange(0, rd, 2, dtype=torch.int64).float() / rd))
    ang = pos.float()[:, None] * inv[None]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b, rest = x[..., :half], x[..., half:rd], x[..., rd:]
    return torch.cat([a * c - b * s, b * c + a * s, rest], -1)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,rd,ps,norm", [(4, 2, 16, 16, 4, True), (6, 2, 32, 32, 8, True), (5, 5, 48, 48, 16, True),
                                                 (8, 2, 128, 128, 16, True), (3, 1, 80, 32, 8, False), (2, 1, 256, 256, 16, True),
                                                 (5, 3, 64, 64, 8, True), (7, 1, 128, 128, 16, False), (9, 3, 32, 32, 4, True)])
@pytest.mark.parametrize("T", [13, 300])
def test_qk_norm_rope_kv(ops, dtype, nh, nkv, hd, rd, ps, norm, T):
    from tandem_b200.config.plan import PositionSpec
    from tandem_b200.parts.rope import RotaryTable

    g = torch.Generator().manual_seed(2)
    pages, eps, theta = -(-(T + 3) // ps) + 4, 1e-5, 12345.0
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, generator=g).to(dtype)
    pos = torch.randint(0, 300, (T,), generator=g, dtype=torch.int32)
    slots = torch.randperm(pages * ps, generator=g)[:T].to(torch.int32)
    slots[3] = -1  # a padding row writes nothing
    qw = (1 + 0.1 * torch.randn(hd, generator=g)) if norm else None
    kw = (1 + 0.1 * torch.randn(hd, generator=g)) if norm else None
    table = RotaryTable(PositionSpec("rope", rotary_dim=rd, theta=theta, max_position=300), "cuda")
    kc = torch.full((pages, nkv, ps, hd), 7.0, dtype=dtype, device="cuda")
    vc = torch.full((pages, nkv, ps, hd), 7.0, dtype=dtype, device="cuda")
    qkv_d = dev(qkv.clone())
    ops.qk_norm_rope_kv(qkv_d, dev(pos), dev(slots), dev(qw) if norm else None, dev(kw) if norm else None, table.cos_sin,
                        kc, vc, nh, nkv, hd, rd, ps, eps)
    x = qkv.float().view(T, nh + 2 * nkv, hd)
    q, k, v = x[:, :nh], x[:, nh:nh + nkv], x[:, nh + nkv:]
    if norm:
        q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + eps) * qw
        k = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + eps) * kw
    q, k = _rope_reference(q, pos, theta, rd), _rope_reference(k, pos, theta, rd)
    out = qkv_d.cpu().float().view(T, nh + 2 * nkv, hd)
    torch.testing.assert_close(out[:, :nh], q, **tol(dtype, 4))
    torch.testing.assert_close(out[:, nh:], x[:, nh:], atol=0, rtol=0)  # k and v columns of qkv stay as they were
    from tandem_b200.cache.layout import to_logical

    kc, vc = to_logical(kc.cpu()).float(), to_logical(vc.cpu()).float()  # undo the physical tile layout
    written = torch.zeros(pages, ps, dtype=torch.bool)
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        written[s // ps, s % ps] = True
        torch.testing.assert_close(kc[s // ps, :, s % ps], k[t], **tol(dtype, 4))
        torch.testing.assert_close(vc[s // ps, :, s % ps], v[t], atol=0, rtol=0)
    assert bool((kc.permute(0, 2, 1, 3)[~written] == 7.0).all()) and bool((vc.permute(0, 2, 1, 3)[~written] == 7.0).all())
    # a run that reads another run's cache writes nothing
    kc2 = torch.zeros((pages, nkv, ps, hd), dtype=dtype, device="cuda")
    ops.qk_norm_rope_kv(dev(qkv.clone()), dev(pos), None, dev(qw) if norm else None, dev(kw) if norm else None,
                        table.cos_sin, None, None, nh, nkv, hd, rd, ps, eps, write_kv=False)
    assert float(kc2.abs().sum()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,I", [(1, 192), (9, 250), (4, 12288), (3, 7)])
def test_silu_mul(ops, dtype, T, I):
    g = torch.Generator().manual_seed(3)
    gu = (torch.randn(T, 2 * I, generator=g) * 2).to(dtype)
    a, b = gu.float()[:, :I], gu.float()[:, I:]
    torch.testing.assert_close(ops.silu_mul(dev(gu)).cpu().float(), a * torch.sigmoid(a) * b, **tol(dtype, 4))


@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (5, 1000, 96), (33, 192, 100), (70, 130, 257), (128, 512, 64), (2, 3, 5)])
def test_gemm_f32_is_true_float32_and_batch_invariant(ops, M, N, K):
    g = torch.Generator().manual_seed(4)
    x, w = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g)
    y = ops.linear(dev(x), dev(w))
    want = (x.double() @ w.double().T)
    assert (y.cpu().double() - want).abs().max() < 1e-5 * math.sqrt(K) * 4
    # TF32 would be off by ~1e-3 here; and a row alone gives bit-identical results
    one = ops.linear(dev(x[M - 1:]), dev(w))
    assert torch.equal(one[0], y[M - 1])


@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (3, 1000, 96), (8, 6144, 4096), (17, 320, 192), (64, 130, 264),
                                   (100, 512, 1024), (300, 1000, 96), (2, 24, 8), (1, 4096, 4096), (5, 24576, 4096),
                                   (64, 4096, 12288), (33, 151936, 512), (16, 128, 64), (32, 129, 72), (48, 4096, 4096),
                                   (7, 100, 100), (65, 256, 256)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_bf16(ops, M, N, K, out_dtype):
    """Up to 64 rows run the tcgen05 weight-streaming kernel (odd N, K that is no multiple of the
    64-element stage, tiles shared between blocks), more rows the library product."""
    g = torch.Generator().manual_seed(5)
    x, w = torch.randn(M, K, generator=g).bfloat16(), (torch.randn(N, K, generator=g) / math.sqrt(K)).bfloat16()
    want = x.double() @ w.double().T
    xd, wd = dev(x), dev(w)
    first = None
    from tandem_b200.kernels import gemm_bf16

    def run():  # the kernel itself wherever it applies, whatever the dispatch would prefer
        if gemm_bf16.skinny_applies(M, N, K):
            return gemm_bf16.skinny(xd, wd, out_dtype)
        return ops.linear(xd, wd, out_dtype=out_dtype)

    torch.testing.assert_close(ops.linear(xd, wd, out_dtype=out_dtype).float(), run().float(), atol=2e-2, rtol=2e-2)
    for attempt in range(2):  # twice: the tile counters must be back at zero, and the sums the same bit for bit
        y = run()
        assert y.dtype == out_dtype and y.shape == (M, N)
        err = (y.cpu().double() - want).abs().max()
        assert err < (2e-2 if out_dtype == torch.bfloat16 else 2e-4 * math.sqrt(K) / 8 + 1e-4), err
        first = y if first is None else first
        assert torch.equal(first, y)
    ops.check_status("cuda")


@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (2, 1000, 96), (1, 4096, 4096), (2, 6144, 4096), (1, 4096, 12288),
                                   (2, 24, 8), (1, 151936, 512), (2, 130, 2056), (1, 7, 2048), (1, 3000, 25600),
                                   (3, 4096, 4096), (4, 1000, 12288), (4, 77, 200), (8, 6144, 4096), (8, 4096, 12288),
                                   (5, 2500, 1000), (8, 17, 72), (7, 24576, 4096), (6, 33, 8200), (7, 100, 20000),
                                   (8, 300, 25600), (9, 6144, 4096), (14, 4096, 4096), (12, 1000, 96), (14, 24576, 4096), (16, 512, 2048),
                                   (13, 77, 200), (16, 17, 72), (11, 2500, 1000), (10, 130, 2056), (11, 300, 5120)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemv_bf16(ops, M, N, K, out_dtype):
    """Up to sixteen rows through the register-streaming kernel: odd N, fewer rows of the weight
    than a block takes, K that is no multiple of a step or of the warps' shares, and the same bits every time."""
    from tandem_b200.kernels import gemm_bf16

    g = torch.Generator().manual_seed(6)
    x, w = torch.randn(M, K, generator=g).bfloat16(), (torch.randn(N, K, generator=g) / math.sqrt(K)).bfloat16()
    want = x.double() @ w.double().T
    xd, wd = dev(x), dev(w)
    assert gemm_bf16.gemv_applies(M, N, K)
    first = gemm_bf16.gemv(xd, wd, out_dtype)
    assert first.dtype == out_dtype and first.shape == (M, N)
    err = (first.cpu().double() - want).abs().max()
    assert err < (2e-2 if out_dtype == torch.bfloat16 else 2e-4 * math.sqrt(K) / 8 + 1e-4), err
    assert torch.equal(first, gemm_bf16.gemv(xd, wd, out_dtype))
    if M > 1:  # a row alone gives the bits it gives beside others
        assert torch.equal(gemm_bf16.gemv(xd[M - 1:].contiguous(), wd, out_dtype)[0], first[M - 1])
    if M > 8:  # and so do the first eight
        assert torch.equal(gemm_bf16.gemv(xd[:8].contiguous(), wd, out_dtype), first[:8])
    assert not gemm_bf16.gemv_applies(17, N, K) and not gemm_bf16.gemv_applies(1, N, K + 4)
    assert gemm_bf16.gemv_applies(8, N, 25600) and not gemm_bf16.gemv_applies(9, N, 25600)  # nine rows of that length do not fit into shared memory
    assert gemm_bf16.gemv_applies(14, N, 4096) and not gemm_bf16.gemv_applies(15, N, 4096)
    assert gemm_bf16.gemv_applies(11, N, 5120) and not gemm_bf16.gemv_applies(12, N, 5120)
    lib = gemm_bf16.load_library("gemv_bf16")
    assert all(bool(lib.tb_gemv_takes(m, k)) == gemm_bf16.gemv_applies(m, N, k) for m in range(0, 18) for k in (8, 72, 2048, 4096, 4100, 5120, 8192, 25600))
    for rows, k in ((17, K), (9, 25600)):
        with pytest.raises(Exception):
            gemm_bf16.gemv(dev(torch.zeros(rows, k).bfloat16()), dev(torch.zeros(8, k).bfloat16()), out_dtype)


@pytest.mark.parametrize("M,I,K", [(1, 16, 64), (8, 12288, 4096), (3, 104, 200), (5, 1000, 1000), (8, 40, 12288), (2, 4096, 520),
                                   (14, 12288, 4096), (9, 104, 200), (16, 1000, 1000)])
def test_gemv_gated_gives_the_bits_of_product_then_activation(ops, M, I, K):
    """silu(x gate^T) * (x up^T) inside the streaming kernel (8 gate rows and their 8 up rows share a
    tile); bit for bit what the product followed by ops.silu_mul gives."""
    from tandem_b200.kernels import gemm_bf16

    g = torch.Generator().manual_seed(8)
    x, w = dev(torch.randn(M, K, generator=g).bfloat16()), dev((torch.randn(2 * I, K, generator=g) / math.sqrt(K) * 3).bfloat16())
    fused = gemm_bf16.gemv(x, w, torch.bfloat16, gated=True)
    assert fused.shape == (M, I)
    plain = ops.silu_mul(gemm_bf16.gemv(x, w, torch.bfloat16))
    assert torch.equal(fused, plain), ((fused.float() - plain.float()).abs().max(), int((fused != plain).sum()))
    gu = x.double().cpu() @ w.double().cpu().T
    want = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
    torch.testing.assert_close(fused.cpu().double(), want, atol=2e-2, rtol=2e-2)  # gate, up and the result are rounded to bfloat16
    with pytest.raises(Exception):
        gemm_bf16.gemv(x, w[: 2 * I - 8].contiguous(), torch.bfloat16, gated=True)  # halves that are no multiple of 8 rows


@pytest.mark.parametrize("M,H,N2,K0", [(1, 4096, 6144, 4096), (8, 4096, 24576, 12288), (5, 1000, 136, 200), (3, 64, 64, 64),
                                        (8, 96, 512, 256), (7, 4096, 4096, 12288), (14, 4096, 24576, 4096), (9, 1000, 136, 200),
                                        (16, 96, 512, 256)])
def test_gemv_takes_the_residual_add_and_the_norm_along(ops, M, H, N2, K0, monkeypatch):
    """A product added into the residual by its own kernel (which also writes residual * norm weight
    and partial sums of squares), and the product behind it scaling its rows by the norm's
    rsqrt(mean square + eps), against the three kernels one after the other: the residual bit for
    bit; the normalised rows (seen through an identity matrix as the second product, float32 out)
    to within the one bfloat16 rounding that has moved; real products within the usual bounds."""
    from tandem_b200.kernels import deferred, gemm_bf16

    if M > 8:  # nine to sixteen rows go to the streaming kernel only where a measurement said so
        monkeypatch.setenv("TANDEM_GEMM", "gemv")
    g = torch.Generator().manual_seed(17 + M)
    x = dev(torch.randn(M, K0, generator=g).bfloat16())
    w1 = dev((torch.randn(H, K0, generator=g) / math.sqrt(K0)).bfloat16())
    res = dev(torch.randn(M, H, generator=g) * 3)
    wn = dev(1 + 0.1 * torch.randn(H, generator=g))
    # one after the other
    res_a = res.clone()
    h_a = ops.add_rmsnorm(gemm_bf16.gemv(x, w1, torch.bfloat16), res_a, wn, 1e-5, torch.bfloat16)
    # the add in the first product's epilogue
    res_b = res.clone()
    pending = ops.add_rmsnorm(deferred.PendingLinear(x, w1), res_b, wn, 1e-5, torch.bfloat16, defer=True)
    assert isinstance(pending, deferred.PendingNorm) and pending.residual is res_b
    assert torch.equal(res_a, res_b)
    assert pending.partials.shape == (pending.parts, 8 if M <= 8 else 16) and (pending.partials[:, M:] == 0).all()
    torch.testing.assert_close(pending.partials.sum(0)[:M].double().cpu(), res_b.double().pow(2).sum(1).cpu(), rtol=1e-5, atol=0)
    assert torch.equal(pending.scaled, (res_b * wn).bfloat16())
    # the scale in the second product's epilogue
    eye = dev(torch.eye(H).bfloat16())
    assert gemm_bf16.scale_fusable(pending, eye)
    h_b = ops.linear(pending, eye, torch.float32)
    assert torch.equal(h_b, ops.linear(pending, eye, torch.float32))  # the same bits every time
    torch.testing.assert_close(h_b, h_a.float(), rtol=2.0 ** -7, atol=1e-30)
    exact = (res_b.double() * torch.rsqrt(res_b.double().pow(2).mean(1, keepdim=True) + 1e-5) * wn.double())
    torch.testing.assert_close(h_b.double(), exact, rtol=2.0 ** -7, atol=1e-30)  # and as close to the true value as the rounded one
    torch.testing.assert_close(deferred.tensor(pending).float(), h_a.float(), rtol=0, atol=0)  # made whole by the norm kernel: its bits
    # a real second product, plain and gated
    w2 = dev((torch.randn(N2, H, generator=g) / math.sqrt(H)).bfloat16())
    want = exact @ w2.double().T
    for out_dtype in (torch.bfloat16, torch.float32):
        torch.testing.assert_close(ops.linear(pending, w2, out_dtype).double(), want, atol=3e-2, rtol=3e-2)
    if N2 % 16 == 0:
        I = N2 // 2
        torch.testing.assert_close(ops.gated_linear(pending, w2).double(), torch.nn.functional.silu(want[:, :I]) * want[:, I:], atol=3e-2, rtol=3e-2)
    # a reader that the streaming kernel does not run gets the rows from the stand-alone norm kernel
    wide_x = deferred.PendingNorm(res_b.repeat(17, 1)[:17].contiguous(), wn, 1e-5, torch.bfloat16, pending.scaled.repeat(17, 1)[:17].contiguous(),
                                  pending.partials, pending.parts)
    w3 = dev((torch.randn(24, H, generator=g) / math.sqrt(H)).bfloat16())
    assert not gemm_bf16.scale_fusable(wide_x, w3) and ops.linear(wide_x, w3).shape == (17, 24)
    ops.check_status("cuda")


# ----------------------------------------------------------------------------- attention
def _paged_case(g, dtype, seqs, nh, nkv, hd, ps, extra_pages=5):
    """seqs: [(start, n)] -> (qkv rows for the new tokens, caches with shuffled pages holding keys 0..start+n-1, ...)."""
    total_pages = sum(-(-(s + n) // ps) for s, n in seqs) + extra_pages
    perm = torch.randperm(total_pages, generator=g).tolist()
    kc = torch.full((total_pages, nkv, ps, hd), float("nan")).to(dtype)  # unwritten slots must never be read
    vc = torch.full((total_pages, nkv, ps, hd), float("nan")).to(dtype)
    width = max(-(-(s + n) // ps) for s, n in seqs)
    table = torch.full((len(seqs), width), -1, dtype=torch.int32)
    K, V, Q, positions, seq_of = [], [], [], [], []
    for b, (start, n) in enumerate(seqs):
        L = start + n
        k = torch.randn(L, nkv, hd, generator=g).to(dtype)
        v = torch.randn(L, nkv, hd, generator=g).to(dtype)
        q = torch.randn(n, nh, hd, generator=g).to(dtype)
        for j in range(-(-L // ps)):
            page = perm.pop()
            table[b, j] = page
            rows = slice(j * ps, min(L, (j + 1) * ps))
            kc[page, :, : rows.stop - rows.start] = k[rows].transpose(0, 1)
            vc[page, :, : rows.stop - rows.start] = v[rows].transpose(0, 1)
        K.append(k), V.append(v), Q.append(q)
        positions += list(range(start, L))
        seq_of += [b] * n
    # the query heads sit in the first nh*hd columns of a wider row, as in the fused projection
    qrows = torch.cat(Q).reshape(len(positions), nh * hd)
    qkv = torch.cat([qrows, torch.zeros(len(positions), 2 * nkv * hd, dtype=dtype)], 1).contiguous()
    return qkv, kc, vc, table, torch.tensor(seq_of, dtype=torch.int32), torch.tensor(positions, dtype=torch.int32), Q, K, V


def phys(cache):
    """A cache filled in logical order -> on the device in the layout the kernels use."""
    from tandem_b200.cache.layout import to_physical

    return to_physical(cache).to("cuda")


def _attention_reference(Q, K, V, seqs, scale, window):
    outs = []
    for (start, n), q, k, v in zip(seqs, Q, K, V):
        q, k, v = q.double(), k.double(), v.double()
        g = q.shape[1] // k.shape[1]
        k, v = k.repeat_interleave(g, 1), v.repeat_interleave(g, 1)
        s = torch.einsum("qhd,khd->hqk", q, k) * scale
        qpos = torch.arange(start, start + n)[:, None]
        kpos = torch.arange(start + n)[None, :]
        ok = kpos <= qpos
        if window:
            ok &= kpos > qpos - window
        s = s.masked_fill(~ok[None], float("-inf"))
        outs.append(torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v).reshape(n, -1))
    return torch.cat(outs)


ATTN_SHAPES = [(4, 2, 16, 4), (6, 2, 32, 8), (5, 5, 48, 16), (8, 2, 128, 16), (3, 1, 80, 8), (10, 2, 64, 16),
               (7, 7, 96, 16), (4, 1, 256, 16), (32, 8, 128, 16)]
ATTN_BATCHES = [[(0, 1)], [(0, 37)], [(40, 1), (3, 1), (129, 1)], [(5, 2), (0, 19), (63, 1), (17, 40)], [(300, 3), (0, 130)]]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,ps", ATTN_SHAPES)
@pytest.mark.parametrize("batch", range(len(ATTN_BATCHES)))
@pytest.mark.parametrize("window", [None, 9])
def test_paged_attention_simt(ops, dtype, nh, nkv, hd, ps, batch, window):
    if (batch + (window or 0) + hd) % 2 and hd not in (16, 128):  # thin the product out
        pytest.skip("covered by the neighbouring cases")
    g = torch.Generator().manual_seed(6 + batch)
    seqs = ATTN_BATCHES[batch]
    qkv, kc, vc, table, seq_of, pos, Q, K, V = _paged_case(g, dtype, seqs, nh, nkv, hd, ps)
    scale = hd ** -0.5
    if window:  # pages wholly behind every query's window may be gone: the kernel must not touch them
        for b, (start, n) in enumerate(seqs):
            for j in range(max(0, start - window + 1) // ps):
                kc[table[b, j]] = float("nan")
                table[b, j] = -1
    out = ops.paged_attention_simt(dev(qkv), phys(kc), phys(vc), dev(table), dev(seq_of), dev(pos), nh, nkv, hd, ps, window, scale)
    want = _attention_reference(Q, K, V, seqs, scale, window)
    torch.testing.assert_close(out.cpu().double(), want, atol=2e-5 if dtype == torch.float32 else 2e-2, rtol=1e-3)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_one_far_key_and_respects_edges(ops, dtype):
    """Random weights hide a wrong key: make one score stand out.  The query at position p is
    aligned with key j only, so the output must be v[j]; j is placed at a page's first and last
    slot, at the far start, at the causal edge and at the window's edge."""
    nh, nkv, hd, ps = 4, 2, 64, 16
    g = torch.Generator().manual_seed(7)
    L = 403
    for j, window in [(0, None), (15, None), (16, None), (399, None), (402, None), (402 - 49, 50), (402 - 50, 50), (387, 100)]:
        seqs = [(L - 1, 1)]
        qkv, kc, vc, table, seq_of, pos, Q, K, V = _paged_case(g, dtype, seqs, nh, nkv, hd, ps)
        direction = torch.randn(hd, generator=g)
        direction /= direction.norm()
        K[0][:] = (0.01 * torch.randn(L, nkv, hd, generator=g)).to(dtype)
        K[0][j] = (8.0 * direction).to(dtype)
        Q[0][:] = (8.0 * direction).to(dtype)
        for p in range(-(-L // ps)):
            rows = slice(p * ps, min(L, (p + 1) * ps))
            kc[table[0, p], :, : rows.stop - rows.start] = K[0][rows].transpose(0, 1)
        qkv[:, : nh * hd] = Q[0].reshape(1, -1)
        out = ops.paged_attention_simt(dev(qkv), phys(kc), phys(vc), dev(table), dev(seq_of), dev(pos), nh, nkv, hd, ps,
                                       window, 1.0).cpu().float().view(nh, hd)
        inside = window is None or j > L - 1 - window
        want = V[0][j].float().repeat_interleave(nh // nkv, 0)
        if inside:
            torch.testing.assert_close(out, want, atol=2e-2, rtol=2e-2)
        else:  # the key lies just outside the window: it must not be seen
            assert (out - want).abs().max() > 0.1



# ----------------------------------------------------------------------------- decode attention (tensor cores)
DECODE_SHAPES = [(4, 2, 16, 4), (6, 2, 32, 8), (5, 5, 48, 16), (32, 8, 128, 16), (3, 1, 80, 8), (10, 2, 64, 16),
                 (8, 8, 64, 32), (4, 1, 256, 16), (20, 1, 64, 16), (6, 3, 128, 4), (2, 1, 112, 2), (12, 4, 96, 1),
                 (14, 2, 128, 8), (9, 3, 64, 48)]
DECODE_BATCHES = [[0], [15], [16], [63, 64, 65], [300, 5, 1000, 129, 0], [2047], [40] * 9]


def _run_decode(qkv, kc, vc, table, nh, nkv, hd, ps, starts, window, scale, target_blocks):
    from tandem_b200.kernels import attention as A
    from tandem_b200.parts.base import KVView

    items = A.plan_decode([(b, b, p) for b, p in enumerate(starts)], window, nkv, target_blocks)
    flat = torch.tensor([x for it in items for x in it] + [0] * (A.ITEM_INTS * 3), dtype=torch.int32)  # spare capacity
    count = torch.tensor([len(items)], dtype=torch.int32)
    kv = KVView(phys(kc), phys(vc), dev(table), None, ps, True)
    return A.paged_attention_decode(dev(qkv), kv, dev(flat), dev(count), nh, nkv, hd, scale), items


@pytest.mark.parametrize("nh,nkv,hd,ps", DECODE_SHAPES)
@pytest.mark.parametrize("batch", range(len(DECODE_BATCHES)))
@pytest.mark.parametrize("window,target", [(None, 592), (None, 8), (70, 4000)])
def test_paged_attention_decode(ops, nh, nkv, hd, ps, batch, window, target):
    if (batch + hd // 16 + (window or 0)) % 3 == 0 and hd not in (64, 128):
        pytest.skip("covered by the neighbouring cases")
    g = torch.Generator().manual_seed(20 + batch)
    starts = DECODE_BATCHES[batch]
    seqs = [(s, 1) for s in starts]
    qkv, kc, vc, table, seq_of, pos, Q, K, V = _paged_case(g, torch.bfloat16, seqs, nh, nkv, hd, ps)
    scale = hd ** -0.5
    if window:
        for b, (start, n) in enumerate(seqs):
            for j in range(max(0, start - window + 1) // ps):
                kc[table[b, j]] = float("nan")
                vc[table[b, j]] = float("nan")
                table[b, j] = -1
    want = _attention_reference(Q, K, V, seqs, scale, window)
    for attempt in range(2):  # twice: the arrival counters must have been put back to zero
        out, items = _run_decode(qkv, kc, vc, table, nh, nkv, hd, ps, starts, window, scale, target)
        torch.testing.assert_close(out.cpu().double(), want, atol=2e-2, rtol=2e-2)
    ops.check_status("cuda")
    if target == 4000 and max(starts) >= 300 and not window:
        assert max(it[5] for it in items) > 1  # the long request was really split


@pytest.mark.parametrize("nh,nkv,hd,ps", [(32, 8, 128, 16), (8, 2, 64, 16), (4, 2, 16, 4), (6, 2, 32, 8), (40, 2, 128, 32), (4, 1, 256, 16),
                                          (8, 4, 64, 2)])
@pytest.mark.parametrize("window,target,norm", [(None, 592, True), (None, 4000, False), (70, 8, True)])
def test_decode_attention_from_the_raw_projection(ops, nh, nkv, hd, ps, window, target, norm):
    """Decode attention that normalises and rotates its query rows and makes each request's newest key
    itself, against the stand-alone kernel followed by decode attention: the same output, the same
    cache, bit for bit.  The stale row it overwrites holds NaN, as does every unwritten slot."""
    from tandem_b200.cache.layout import to_logical
    from tandem_b200.kernels import attention as A
    from tandem_b200.parts.base import KVView

    g = torch.Generator().manual_seed(31 + hd)
    starts = [0, 15, 16, 63, 64, 200, 641, 1500][: 5 if hd == 256 else 8]
    seqs = [(s, 1) for s in starts]
    _, kc, vc, table, seq_of, pos, Q, K, V = _paged_case(g, torch.bfloat16, seqs, nh, nkv, hd, ps)
    T = len(starts)
    raw = torch.randn(T, (nh + 2 * nkv) * hd, generator=g).bfloat16()
    slots = torch.tensor([int(table[b, s // ps]) * ps + s % ps for b, s in enumerate(starts)], dtype=torch.int32)
    for b, s in enumerate(starts):  # the new token's row has not been written yet
        kc[table[b, s // ps], :, s % ps] = float("nan")
        vc[table[b, s // ps], :, s % ps] = float("nan")
    if window:
        for b, s in enumerate(starts):
            for j in range(max(0, s - window + 1) // ps):
                kc[table[b, j]] = float("nan")
                vc[table[b, j]] = float("nan")
                table[b, j] = -1
    qw = dev(1 + 0.1 * torch.randn(hd, generator=g)) if norm else None
    kw = dev(1 + 0.1 * torch.randn(hd, generator=g)) if norm else None
    cos_sin = dev(torch.randn(2000, hd, generator=g))
    items = A.plan_decode([(b, b, p) for b, p in enumerate(starts)], window, nkv, target)
    flat = dev(torch.tensor([x for it in items for x in it], dtype=torch.int32))
    count = dev(torch.tensor([len(items)], dtype=torch.int32))
    scale = hd ** -0.5
    assert A.fresh_applies(hd, hd, True)

    def run(fresh):
        kv = KVView(phys(kc), phys(vc), dev(table), dev(slots), ps, True)
        qkv = dev(raw.clone())
        if fresh:
            out = A.paged_attention_decode(qkv, kv, flat, count, nh, nkv, hd, scale,
                                           fresh=dict(positions=dev(pos), slots=kv.slots, q_norm=qw, k_norm=kw, cos_sin=cos_sin, eps=1e-5))
        else:
            ops.qk_norm_rope_kv(qkv, dev(pos), kv.slots, qw, kw, cos_sin, kv.k, kv.v, nh, nkv, hd, hd, ps, 1e-5)
            out = A.paged_attention_decode(qkv, kv, flat, count, nh, nkv, hd, scale)
        return out, to_logical(kv.k), to_logical(kv.v)

    o1, k1, v1 = run(False)
    o2, k2, v2 = run(True)
    assert not torch.isnan(o1).any()
    assert torch.equal(o1, o2), (o1.float() - o2.float()).abs().max()
    written = torch.zeros(k1.shape[0], ps, dtype=torch.bool)
    for b, s in enumerate(starts):
        written[table[b, s // ps], s % ps] = True
    assert torch.equal(k1.cpu()[written.nonzero(as_tuple=True)[0], :, written.nonzero(as_tuple=True)[1]],
                       k2.cpu()[written.nonzero(as_tuple=True)[0], :, written.nonzero(as_tuple=True)[1]])
    assert torch.equal(v1.cpu()[written.nonzero(as_tuple=True)[0], :, written.nonzero(as_tuple=True)[1]],
                       v2.cpu()[written.nonzero(as_tuple=True)[0], :, written.nonzero(as_tuple=True)[1]])
    assert not torch.isnan(k2.cpu()[written.nonzero(as_tuple=True)[0], :, written.nonzero(as_tuple=True)[1]].float()).any()
    ops.check_status("cuda")


def test_decode_finds_one_far_key(ops):
    nh, nkv, hd, ps = 8, 2, 128, 16
    g = torch.Generator().manual_seed(21)
    L = 1500
    for j, window in [(0, None), (15, None), (16, None), (63, None), (64, None), (1499, None), (1498, None), (1000, 501),
                      (999, 501)]:
        seqs = [(L - 1, 1)]
        qkv, kc, vc, table, seq_of, pos, Q, K, V = _paged_case(g, torch.bfloat16, seqs, nh, nkv, hd, ps)
        direction = torch.randn(hd, generator=g)
        direction /= direction.norm()
        K[0][:] = (0.01 * torch.randn(L, nkv, hd, generator=g)).bfloat16()
        K[0][j] = (8.0 * direction).bfloat16()
        for p in range(-(-L // ps)):
            rows = slice(p * ps, min(L, (p + 1) * ps))
            kc[table[0, p], :, : rows.stop - rows.start] = K[0][rows].transpose(0, 1)
        qkv[:, : nh * hd] = (8.0 * direction).bfloat16().repeat(nh)
        out, _ = _run_decode(qkv, kc, vc, table, nh, nkv, hd, ps, [L - 1], window, 1.0, 4000)
        out = out.cpu().float().view(nh, hd)
        want = V[0][j].float().repeat_interleave(nh // nkv, 0)
        if window is None or j > L - 1 - window:
            torch.testing.assert_close(out, want, atol=2e-2, rtol=2e-2)
        else:
            assert (out - want).abs().max() > 0.1
    ops.check_status("cuda")



# ----------------------------------------------------------------------------- prefill attention (tensor cores)
PREFILL_BATCHES = ATTN_BATCHES + [[(0, 64)], [(0, 65), (100, 31)], [(7, 200)], [(1000, 17), (0, 300), (63, 2)]]


@pytest.mark.parametrize("nh,nkv,hd,ps", DECODE_SHAPES)
@pytest.mark.parametrize("batch", range(len(PREFILL_BATCHES)))
@pytest.mark.parametrize("window", [None, 9, 70])
@pytest.mark.parametrize("impl", ["tcgen05", "mma"])
def test_paged_attention_prefill(ops, monkeypatch, nh, nkv, hd, ps, batch, window, impl):
    from tandem_b200.kernels import attention as A
    from tandem_b200.parts.base import KVView

    if (batch + hd // 16 + (window or 0)) % 3 == 0 and hd not in (64, 128):
        pytest.skip("covered by the neighbouring cases")
    monkeypatch.setenv("TANDEM_PREFILL", impl)
    if impl == "tcgen05" and not A.tcgen05_prefill_applies(hd, ps):
        pytest.skip("the tcgen05 kernel does not take this head size or page size")
    g = torch.Generator().manual_seed(30 + batch)
    seqs = PREFILL_BATCHES[batch]
    qkv, kc, vc, table, seq_of, pos, Q, K, V = _paged_case(g, torch.bfloat16, seqs, nh, nkv, hd, ps)
    scale = hd ** -0.5
    if window:
        for b, (start, n) in enumerate(seqs):
            for j in range(max(0, start - window + 1) // ps):
                kc[table[b, j]] = float("nan")
                vc[table[b, j]] = float("nan")
                table[b, j] = -1
    rows, at = [], 0
    for b, (start, n) in enumerate(seqs):
        rows.append((at, b, start, n))
        at += n
    plan = A.prefill_plan(rows, nh, nkv, hd, ps, window, "cuda")
    tokens_planned = plan[..., 3].sum().item() // nkv if plan.dim() == 3 else plan.view(-1, 4)[:, 3].sum().item()
    assert tokens_planned == at
    kv = KVView(phys(kc), phys(vc), dev(table), None, ps, True)
    out = A.paged_attention_prefill(dev(qkv), kv, plan, nh, nkv, hd, window, scale)
    want = _attention_reference(Q, K, V, seqs, scale, window)
    torch.testing.assert_close(out.cpu().double(), want, atol=2e-2, rtol=2e-2)
    ops.check_status("cuda")


@pytest.mark.parametrize("impl", ["tcgen05", "mma"])
def test_prefill_finds_one_far_key_per_row(ops, monkeypatch, impl):
    """Every query row is aligned with one key of its own (far back, at a page edge, at the causal
    edge, at the window's edge): its output must be that key's value."""
    from tandem_b200.kernels import attention as A
    from tandem_b200.parts.base import KVView

    monkeypatch.setenv("TANDEM_PREFILL", impl)
    nh, nkv, hd, ps = 8, 2, 128, 16
    g = torch.Generator().manual_seed(31)
    start, n = 700, 90
    L = start + n
    for window in (None, 300):
        seqs = [(start, n)]
        qkv, kc, vc, table, seq_of, pos, Q, K, V = _paged_case(g, torch.bfloat16, seqs, nh, nkv, hd, ps)
        dirs = torch.randn(n, hd, generator=g)
        dirs /= dirs.norm(dim=-1, keepdim=True)
        K[0][:] = (0.01 * torch.randn(L, nkv, hd, generator=g)).bfloat16()
        target = []
        for i in range(n):
            q = start + i
            lo = 0 if window is None else q - window + 1
            j = [lo, q, (q // ps) * ps, max(lo, (q // ps) * ps - 1), lo + (q - lo) // 2][i % 5]
            # keys already taken by an earlier row of this test would pull two rows: move on to a free one
            while j in target and j < q:
                j += 1
            target.append(j)
            K[0][j] = K[0][j] + (8.0 * dirs[i]).bfloat16()[None, :]
            Q[0][i] = (8.0 * dirs[i]).bfloat16()[None, :].expand(nh, hd)
        for p in range(-(-L // ps)):
            rows = slice(p * ps, min(L, (p + 1) * ps))
            kc[table[0, p], :, : rows.stop - rows.start] = K[0][rows].transpose(0, 1)
        qkv[:, : nh * hd] = Q[0].reshape(n, -1)
        kv = KVView(phys(kc), phys(vc), dev(table), None, ps, True)
        out = A.paged_attention_prefill(dev(qkv), kv, A.prefill_plan([(0, 0, start, n)], nh, nkv, hd, ps, window, "cuda"),
                                        nh, nkv, hd, window, 1.0).cpu().float().view(n, nh, hd)
        ok = 0
        for i, j in enumerate(target):
            if target.count(j) == 1:
                torch.testing.assert_close(out[i], V[0][j].float().repeat_interleave(nh // nkv, 0), atol=3e-2, rtol=3e-2)
                ok += 1
        assert ok > n // 2
    ops.check_status("cuda")


# ----------------------------------------------------------------------------- sampling
@pytest.mark.parametrize("R,V", [(1, 10), (3, 1000), (5, 151936), (2, 777)])
def test_argmax(ops, R, V):
    g = torch.Generator().manual_seed(8)
    x = torch.randn(R, V, generator=g)
    x[0, V // 2] = x[0, V - 1] = 99.0  # equal maxima: the lowest index
    got = ops.argmax(dev(x)).cpu()
    assert got.dtype == torch.int32 and got.tolist() == x.argmax(-1).tolist() and got[0] == V // 2


def _sample_reference(logits, temperature, top_k, top_p, min_p, u):
    import plain_qwen3 as plain

    p = plain.filtered_probs(logits, temperature, top_k, top_p, min_p)
    return plain.inverse_cdf_draw(p, u), p


@pytest.mark.parametrize("V", [50, 1000, 151936])
def test_sample_matches_the_plain_sampler(ops, V):
    g = torch.Generator().manual_seed(9)
    rows = [dict(t=1.0, k=-1, p=1.0, m=0.0), dict(t=0.7, k=5, p=1.0, m=0.0), dict(t=1.3, k=-1, p=0.8, m=0.0),
            dict(t=0.9, k=-1, p=1.0, m=0.2), dict(t=0.8, k=40, p=0.9, m=0.05), dict(t=0.0, k=3, p=0.5, m=0.1),
            dict(t=2.0, k=1, p=1.0, m=0.0)]
    for trial in range(4):
        R = len(rows)
        logits = torch.randn(R, V, generator=g) * 3
        u = torch.rand(R, generator=g)
        got = ops.sample(dev(logits), dev(torch.tensor([r["t"] for r in rows])),
                         dev(torch.tensor([r["k"] for r in rows], dtype=torch.int32)),
                         dev(torch.tensor([r["p"] for r in rows])), dev(torch.tensor([r["m"] for r in rows])),
                         dev(u)).cpu().tolist()
        for i, r in enumerate(rows):
            if r["t"] < 1e-5:
                assert got[i] == int(logits[i].argmax())
                continue
            want, p = _sample_reference(logits[i], r["t"], r["k"], r["p"], r["m"], float(u[i]))
            if got[i] != want:  # only where u * total falls within rounding of a boundary of the CDF
                cum = p.cumsum(-1)
                target = float(u[i]) * float(cum[-1])
                lo = float(cum[got[i]] - p[got[i]])
                assert p[got[i]] > 0 and lo - 1e-5 <= target <= float(cum[got[i]]) + 1e-5, (i, trial, got[i], want)


@pytest.mark.parametrize("V", [151936, 1003])
def test_sample_does_not_depend_on_the_number_of_rows(ops, V):
    """A row's blocks share eight chunks of the vocabulary however many they are (eight blocks a row for
    few rows, fewer for many): floating-point sums are taken per chunk, so the token of a row is the
    same alone, among 20 rows, among 70 and among 200."""
    g = torch.Generator().manual_seed(31)
    R = 200
    logits = dev(torch.randn(R, V, generator=g) * 3)
    t = dev(0.5 + torch.rand(R, generator=g))
    k = dev(torch.where(torch.rand(R, generator=g) < 0.5, torch.randint(1, 100, (R,), generator=g), torch.full((R,), -1)).to(torch.int32))
    p = dev(torch.where(torch.rand(R, generator=g) < 0.5, 0.5 + 0.5 * torch.rand(R, generator=g), torch.ones(R)))
    m = dev(torch.where(torch.rand(R, generator=g) < 0.3, 0.1 * torch.rand(R, generator=g), torch.zeros(R)))
    u = dev(torch.rand(R, generator=g))
    whole = ops.sample(logits, t, k, p, m, u)
    assert torch.equal(whole, ops.sample(logits, t, k, p, m, u))
    for n in (1, 20, 70):
        part = ops.sample(logits[:n].contiguous(), t[:n].contiguous(), k[:n].contiguous(), p[:n].contiguous(), m[:n].contiguous(),
                          u[:n].contiguous())
        assert torch.equal(part, whole[:n]), n


def test_sample_keeps_only_filtered_tokens_and_follows_u(ops):
    V = 4
    logits = torch.log(torch.tensor([[0.5, 0.3, 0.15, 0.05]])).repeat(6, 1)
    one, none = torch.ones(6), torch.zeros(6)
    k = torch.tensor([2, 2, -1, -1, -1, -1], dtype=torch.int32)
    p = torch.tensor([1.0, 1.0, 0.7, 0.7, 1.0, 1.0])
    m = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.5, 0.5])
    u = torch.tensor([0.62, 0.63, 0.62, 0.63, 0.62, 0.999])
    got = ops.sample(dev(logits), dev(one), dev(k), dev(p), dev(m), dev(u)).cpu().tolist()
    assert got == [0, 1, 0, 1, 0, 1]  # every filter leaves [.625, .375, 0, 0]
    u = torch.tensor([0.0, 0.49, 0.51, 0.79, 0.81, 0.96])
    got = ops.sample(dev(logits), dev(one), dev(torch.full((6,), -1, dtype=torch.int32)), dev(one), dev(none), dev(u))
    assert got.cpu().tolist() == [0, 0, 1, 1, 2, 3]


def test_refusals(ops):
    x = torch.zeros(2, 8)
    with pytest.raises(ops.KernelError, match="CUDA"):
        ops.silu_mul(x)  # no CPU path
    with pytest.raises(ops.KernelError, match="float32 or bfloat16"):
        ops.silu_mul(dev(x.half()))
    with pytest.raises(ops.KernelError):
        ops.linear(dev(x), dev(torch.zeros(4, 7)))
    with pytest.raises(ops.KernelError, match="share"):
        ops.paged_attention_simt(dev(torch.zeros(1, 96)), dev(torch.zeros(1, 2, 4, 16)), dev(torch.zeros(1, 2, 4, 16)),
                                 dev(torch.zeros(1, 1, dtype=torch.int32)), dev(torch.zeros(1, dtype=torch.int32)),
                                 dev(torch.zeros(1, dtype=torch.int32)), 3, 2, 16, 4, None, 1.0)


# ----------------------------------------------------------------------------- long contexts
@pytest.mark.parametrize("hd,ps,window", [(128, 16, None), (128, 16, 3000), (64, 8, None), (48, 16, None)])
def test_attention_over_more_pages_than_the_kernels_cache(ops, hd, ps, window):
    """A context of 9,000 keys on pages of 8 or 16 has more pages than a block keeps in shared
    memory (512): the kernels then read the block table from global memory.  A portion of 150
    tokens at the end (prefill kernels) and one decoded token (decode kernel, cut into items);
    with a window, the pages in front of it are given back and hold NaN."""
    from tandem_b200.kernels import attention as A
    from tandem_b200.parts.base import KVView

    nh, nkv = 4, 2
    g = torch.Generator().manual_seed(50 + hd)
    start, n = 8850, 150
    seqs = [(start, n)]
    qkv, kc, vc, table, seq_of, pos, Q, K, V = _paged_case(g, torch.bfloat16, seqs, nh, nkv, hd, ps)
    assert table.shape[1] > 512
    scale = hd ** -0.5
    if window:
        for j in range((start - window + 1) // ps):  # pages that lie before every query's window are given back
            kc[table[0, j]] = float("nan")
            vc[table[0, j]] = float("nan")
            table[0, j] = -1
    kv = KVView(phys(kc), phys(vc), dev(table), None, ps, True)
    want = _attention_reference(Q, K, V, seqs, scale, window)
    for impl in ("tcgen05", "mma"):
        if impl == "tcgen05" and not A.tcgen05_prefill_applies(hd, ps):
            continue
        import os
        os.environ["TANDEM_PREFILL"] = impl
        try:
            out = A.paged_attention_prefill(dev(qkv), kv, A.prefill_plan([(0, 0, start, n)], nh, nkv, hd, ps, window, "cuda"),
                                            nh, nkv, hd, window, scale)
        finally:
            os.environ.pop("TANDEM_PREFILL", None)
        torch.testing.assert_close(out.cpu().double(), want, atol=2e-2, rtol=2e-2)
    # the last token alone through the decode kernel, its keys cut into items
    L = start + n
    items = A.plan_decode([(0, 0, L - 1)], window, nkv)
    assert len(items) > 1
    flat = torch.tensor([x for it in items for x in it], dtype=torch.int32)
    out = A.paged_attention_decode(dev(qkv[-1:].contiguous()), kv, dev(flat), dev(torch.tensor([len(items)], dtype=torch.int32)),
                                   nh, nkv, hd, scale)
    torch.testing.assert_close(out.cpu().double(), want[-1:], atol=2e-2, rtol=2e-2)
    ops.check_status("cuda")


# ----------------------------------------------------------------------------- the many-row tcgen05 product
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (300, 520, 200), (2048, 4096, 4096), (1, 8, 8), (129, 6144, 1024), (1000, 1000, 72)])
@pytest.mark.parametrize("out", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("impl", ["wide", "wide_pair"])
def test_gemm_wide(ops, M, N, K, out, impl):
    from tandem_b200.kernels import gemm_bf16

    g = torch.Generator().manual_seed(60 + M)
    x = (torch.randn(M, K, generator=g)).bfloat16()
    w = (torch.randn(N, K, generator=g) * K ** -0.5).bfloat16()
    y = getattr(gemm_bf16, impl)(dev(x), dev(w), out)
    want = dev(x).float() @ dev(w).float().T  # float32 products of bfloat16 operands, float32 sums
    torch.testing.assert_close(y.float(), want, **(dict(atol=2e-2, rtol=2e-2) if out == torch.bfloat16 else dict(atol=2e-3, rtol=2e-3)))
    ops.check_status("cuda")


@pytest.mark.parametrize("M,I,K", [(128, 128, 64), (300, 264, 200), (2048, 1536, 4096), (3, 8, 16), (17, 17408, 5120), (40, 1000, 520)])
@pytest.mark.parametrize("impl", ["wide", "wide_pair"])
def test_gemm_wide_gated(ops, M, I, K, impl):
    """Rows [gate | up] of the weight in one launch: silu(x gate^T) * (x up^T), both products rounded
    to bfloat16 first, as the separate kernels round them."""
    from tandem_b200.kernels import gemm_bf16

    g = torch.Generator().manual_seed(70 + M)
    x = dev((torch.randn(M, K, generator=g)).bfloat16())
    w = dev((torch.randn(2 * I, K, generator=g) * K ** -0.5).bfloat16())
    y = getattr(gemm_bf16, impl)(x, w, torch.bfloat16, gated=True)
    gu = (x.float() @ w.float().T).bfloat16().float()
    want = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
    torch.testing.assert_close(y.float(), want, atol=2e-2, rtol=2e-2)
    ops.check_status("cuda")
