"""tcgen05 bf16x3 matrix products (through the C ABI) against float64 torch.matmul.
Tolerance: 1e-4 relative Frobenius error (measured: ~1e-5)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 1e-4


def rel(a, b):
    return float((a.double() - b).norm() / b.norm())


def device_ok(lib):
    torch.cuda.synchronize()
    return lib.qt_device_error(1) == 0


@pytest.mark.parametrize("trans_a,trans_b", [(False, True), (False, False), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 128, 192), (100, 72, 50), (672, 672, 336), (1200, 1200, 768)])
def test_matmul_all_majors(native_lib, trans_a, trans_b, M, N, K):
    from optimizers import _gemm
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N * 3 + K)
    b = 2
    A = torch.randn((b, K, M) if trans_a else (b, M, K), device="cuda", generator=g)
    B = torch.randn((b, N, K) if trans_b else (b, K, N), device="cuda", generator=g)
    D, _ = _gemm.matmul(_gemm.split(A), _gemm.split(B), trans_a=trans_a, trans_b=trans_b)
    assert device_ok(native_lib)
    ref = (A.transpose(1, 2) if trans_a else A).double() @ (B.transpose(1, 2) if trans_b else B).double()
    assert rel(D, ref) < TOL, rel(D, ref)


def test_alpha_beta_c_and_plane_output(native_lib):
    from optimizers import _gemm
    g = torch.Generator(device="cuda").manual_seed(5)
    b, M, N, K = 3, 200, 328, 136
    A = torch.randn(b, M, K, device="cuda", generator=g)
    B = torch.randn(b, K, N, device="cuda", generator=g)
    C = torch.randn(b, M, N, device="cuda", generator=g)
    D, P = _gemm.matmul(_gemm.split(A), _gemm.split(B), alpha=-0.5, beta=1.5, C=C, want_planes=True, out_bound=100.0)
    assert device_ok(native_lib)
    ref = -0.5 * (A.double() @ B.double()) + 1.5 * C.double()
    assert rel(D, ref) < TOL
    assert rel(P.to_float(), ref) < TOL
    # output canary: a padded output buffer keeps its guard columns
    big = torch.full((b, M, N + 8), 7.0, device="cuda")
    _gemm.matmul(_gemm.split(A), _gemm.split(B), out=big[:, :, :N])
    assert device_ok(native_lib)
    assert bool((big[:, :, N:] == 7.0).all())
    assert rel(big[:, :, :N], A.double() @ B.double()) < TOL


def test_split_planes_precision(native_lib):
    """bf16 planes: every element to 16 significant bits.  Scaled fp16 planes: 22 significant bits
    for every element within 2^12 of the matrix's largest one, and an absolute error below
    2^-33 of the largest element for the rest (columns here span six decades)."""
    from optimizers import _gemm
    X = torch.randn(2, 77, 130, device="cuda") * torch.logspace(-3, 3, 130, device="cuda")
    P = _gemm.split_bf16(X)
    err = (P.to_float() - X).abs() / X.abs().clamp_min(1e-30)
    assert float(err.max()) < 2.0 ** -15
    H = _gemm.split(X)
    assert H.f16 and H.exp is not None
    amax = X.abs().amax(dim=(1, 2), keepdim=True)
    scaled_max = amax.squeeze() * torch.exp2(H.exp.float())
    assert bool((scaled_max < 2.0 ** _gemm.SPLIT_TARGET).all()) and bool((scaled_max >= 2.0 ** (_gemm.SPLIT_TARGET - 1)).all())
    err = (H.to_float() - X).abs()
    assert bool((err <= torch.maximum(X.abs() * 2.0 ** -21, amax * 2.0 ** -32)).all())
    assert device_ok(native_lib)


@pytest.mark.parametrize("trans_a,trans_b", [(False, False), (True, False), (False, True)])
def test_matmul_f32_entry_point_with_caller_scratch(native_lib, trans_a, trans_b):
    """qt_matmul_f32: fp32 operands, planes built in caller-provided scratch memory."""
    import ctypes as ct
    lib = native_lib
    g = torch.Generator(device="cuda").manual_seed(17)
    b, M, N, K = 3, 320, 200, 456
    A = torch.randn((b, K, M) if trans_a else (b, M, K), device="cuda", generator=g)
    B = torch.randn((b, N, K) if trans_b else (b, K, N), device="cuda", generator=g)
    C = torch.randn(b, M, N, device="cuda", generator=g)
    D = torch.empty(b, M, N, device="cuda")
    need = lib.qt_matmul_f32_scratch_bytes(M, N, K, b, int(trans_a), int(trans_b))
    scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
    P = lambda t: ct.c_void_p(t.data_ptr())
    st = ct.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.qt_matmul_f32(P(A), A.stride(1), A.stride(0), int(trans_a), P(B), B.stride(1), B.stride(0), int(trans_b),
                           M, N, K, b, 2.0, -1.0, P(C), N, M * N, P(D), N, M * N, P(scratch), need, st)
    assert rc == 0 and device_ok(lib)
    ref = 2.0 * ((A.transpose(1, 2) if trans_a else A).double() @ (B.transpose(1, 2) if trans_b else B).double()) - C.double()
    assert rel(D, ref) < TOL
    # too little scratch is refused before anything is launched
    assert lib.qt_matmul_f32(P(A), A.stride(1), A.stride(0), int(trans_a), P(B), B.stride(1), B.stride(0), int(trans_b),
                             M, N, K, b, 1.0, 0.0, None, 0, 0, P(D), N, M * N, P(scratch), need - 4096, st) == 1


@pytest.mark.parametrize("trans_a,trans_b", [(False, True), (True, False), (False, False)])
def test_three_plane_product_reaches_fp32_accuracy(native_lib, trans_a, trans_b):
    """hi/mid/lo planes, six MMAs per k-slice: at least as accurate as an fp32 library product."""
    from optimizers import _gemm
    g = torch.Generator(device="cuda").manual_seed(31)
    b, M, N, K = 2, 328, 264, 1200
    A = torch.randn((b, K, M) if trans_a else (b, M, K), device="cuda", generator=g)
    B = torch.randn((b, N, K) if trans_b else (b, K, N), device="cuda", generator=g)
    C = torch.randn(b, M, N, device="cuda", generator=g)
    D, _ = _gemm.matmul(_gemm.split3(A), _gemm.split3(B), trans_a=trans_a, trans_b=trans_b, alpha=0.05, beta=0.95, C=C)
    assert device_ok(native_lib)
    opA = A.transpose(1, 2) if trans_a else A
    opB = B.transpose(1, 2) if trans_b else B
    ref = 0.05 * (opA.double() @ opB.double()) + 0.95 * C.double()
    fp32 = torch.baddbmm(C, opA, opB, beta=0.95, alpha=0.05)
    assert rel(D, ref) < 2e-6, rel(D, ref)               # measured 8e-7, independent of K
    assert rel(D, ref) < 4 * rel(fp32, ref) + 1e-6
    P = _gemm.split3(A)
    back = (P.hi.float() + P.mid.float() + P.lo.float()).view(b, A.shape[1], P.ld)[:, :, : A.shape[2]]   # rows are padded to the pitch
    assert float((back - A).abs().max() / A.abs().max()) < 2.0 ** -22


def _state(b, n, device, diagreal):
    nb = (n + 63) // 64
    row_bytes = ((n * n + 1) // 2 + 15) // 16 * 16
    var = torch.zeros(b, row_bytes, dtype=torch.uint8, device=device)
    absmax = torch.zeros(b, n * nb, device=device)
    diag = torch.zeros(b, n, device=device) if diagreal else None
    return var, absmax, diag


def _quantize_batch(lib, X, code, st):
    import ctypes as ct
    b, n, _ = X.shape
    var, absmax, diag = st
    p = lambda t: None if t is None else ct.c_void_p(t.data_ptr())
    rc = lib.qt_quantize_blockwise(p(X), 0, n * n, p(code), n, b, p(absmax), absmax.stride(0), p(diag), n,
                                   p(var), var.stride(0), 64, 4, ct.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0


def _dequantize_batch(lib, st, code, n):
    import ctypes as ct
    var, absmax, diag = st
    b = var.shape[0]
    out = torch.empty(b, n, n, device=var.device)
    p = lambda t: None if t is None else ct.c_void_p(t.data_ptr())
    rc = lib.qt_dequantize_blockwise(p(var), var.stride(0), p(code), n, b, p(absmax), absmax.stride(0), p(diag), n,
                                     p(out), 0, n * n, 64, 4, ct.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    return out


@pytest.mark.parametrize("encoding", ["f16x2", "bf16x3"])
@pytest.mark.parametrize("n,k,axis,diagreal,with_old", [
    (128, 64, 0, True, True), (512, 384, 1, True, True), (1200, 768, 0, True, True), (1200, 3072, 1, False, True),
    (672, 768, 0, True, False), (1104, 200, 1, False, True), (2048, 2048, 0, True, True), (16, 40, 0, True, True),
    (48, 48, 1, False, True)])
def test_quantizing_epilogue_equals_unfused_sequence(native_lib, n, k, axis, diagreal, with_old, encoding):
    """state <- quantize(w2 * G G^T + w1 * dequantize(state)) inside the GEMM epilogue: the code
    bytes, block scales and diagonal must equal dequantize -> product -> quantize bit for bit (same
    operand planes: scaled fp16 pairs as the optimizers use them, or three bf16 planes), and the
    dequantized result must be within 4-bit quantization error of the float64 value."""
    import qtensor.functional as F
    from optimizers import _gemm
    dev = "cuda"
    b = 3
    gen = torch.Generator(device=dev).manual_seed(n * 31 + k)
    code = F.create_linear_map(True, 4, 2).to(dev)
    G = torch.randn((b, n, k) if axis == 0 else (b, k, n), device=dev, generator=gen) / n ** 0.5
    # old state: SPD with a wide spectrum, one matrix left at zero (all-zero blocks)
    Q = torch.linalg.qr(torch.randn(b, n, n, device=dev, generator=gen)).Q
    lam = torch.exp(torch.rand(b, n, device=dev, generator=gen) * 13.8 - 13.8)
    L0 = (Q * lam[:, None, :]) @ Q.transpose(1, 2)
    L0 = 0.5 * (L0 + L0.transpose(1, 2))
    L0[1].zero_()
    old = _state(b, n, dev, diagreal)
    _quantize_batch(native_lib, L0.contiguous(), code, old)
    w1, w2 = 0.95, 0.05
    P = _gemm.split(G) if encoding == "f16x2" else _gemm.split3(G)
    ta, tb = (False, True) if axis == 0 else (True, False)
    # unfused sequence
    Lold = _dequantize_batch(native_lib, old, code, n) if with_old else None
    D, _ = _gemm.matmul(P, P, trans_a=ta, trans_b=tb, alpha=w2, beta=w1 if with_old else 0.0, C=Lold)
    want = _state(b, n, dev, diagreal)
    _quantize_batch(native_lib, D, code, want)
    # fused, written to a fresh state and then in place
    got = _state(b, n, dev, diagreal)
    _gemm.matmul_q4(P, P, code, got, trans_a=ta, trans_b=tb, alpha=w2, beta=w1, old=old if with_old else None)
    assert device_ok(native_lib)
    nbytes = (n * n + 1) // 2
    for w, g_, name in zip(want, got, ("codes", "absmax", "diag")):
        if w is None:
            continue
        w, g_ = (w[:, :nbytes], g_[:, :nbytes]) if name == "codes" else (w, g_)
        assert torch.equal(w.view(torch.uint8 if name == "codes" else torch.int32),
                           g_.view(torch.uint8 if name == "codes" else torch.int32)), name
    if with_old:
        _gemm.matmul_q4(P, P, code, old, trans_a=ta, trans_b=tb, alpha=w2, beta=w1, old=old)
        assert device_ok(native_lib)
        assert torch.equal(old[0][:, :nbytes], want[0][:, :nbytes]) and torch.equal(old[1], want[1])
    Gd = G.double()
    ref = w2 * (Gd @ Gd.transpose(1, 2) if axis == 0 else Gd.transpose(1, 2) @ Gd)
    if with_old:
        ref = ref + w1 * Lold.double()
    assert rel(D, ref) < 2e-6, rel(D, ref)                # both encodings are fp32-grade


def test_fp16_plane_products_reach_fp32_accuracy(native_lib):
    """Scaled fp16 planes (22 bits) with 128-k accumulation chains against float64, next to the
    same product from bf16 planes (16 bits, one chain) and from an fp32 library product: chained
    plane outputs (explicit bound, worst-case exponent) and a large common scale included."""
    from optimizers import _gemm
    g = torch.Generator(device="cuda").manual_seed(41)
    b, M, N, K = 2, 300, 520, 1200
    A = torch.randn(b, M, K, device="cuda", generator=g) * 3e4          # scales far from 1 on purpose
    B = torch.randn(b, K, N, device="cuda", generator=g) * 2e-5
    ref = A.double() @ B.double()
    D16, _ = _gemm.matmul(_gemm.split(A), _gemm.split(B))
    Dbf, _ = _gemm.matmul(_gemm.split_bf16(A), _gemm.split_bf16(B))
    assert device_ok(native_lib)
    e16, ebf, e32 = rel(D16, ref), rel(Dbf, ref), rel(torch.bmm(A, B), ref)
    print(f"fp16x2 {e16:.2e}  bf16x2 {ebf:.2e}  fp32 library {e32:.2e}")
    assert e16 < 2e-6 and e16 < 4 * e32 + 1e-6 and ebf < 1e-4
    # plane outputs: worst-case exponent, then consumed by a second product
    _, P = _gemm.matmul(_gemm.split(A), _gemm.split(B), want_float=False, want_planes=True)
    assert rel(P.to_float(), ref) < 2e-6
    C = torch.randn(b, N, 200, device="cuda", generator=g)
    D2, _ = _gemm.matmul(P, _gemm.split(C))
    assert device_ok(native_lib)
    assert rel(D2, ref @ C.double()) < 3e-6
    # explicit bound that is too small: the planes clamp and the sticky error word reports it
    _gemm.matmul(_gemm.split(A), _gemm.split(B), want_float=False, want_planes=True, out_bound=1e-3)
    torch.cuda.synchronize()
    assert native_lib.qt_device_error(1) == 9


def test_split_rows_gathers_and_scales(native_lib):
    """qt_split_bf16_rows == split(scale[:, :, None] * X[gathered rows]) bit for bit, wide and scalar variants."""
    from optimizers import _gemm
    g = torch.Generator(device="cuda").manual_seed(11)
    for cols in (768, 100):
        X = torch.randn(3, 40, cols, device="cuda", generator=g)
        idx = torch.stack([torch.randperm(40, device="cuda", generator=g)[:17] for _ in range(3)])
        w = torch.rand(3, 17, device="cuda", generator=g) + 0.5
        for index, scale in ((idx, w), (idx, None), (None, torch.rand(3, 40, device="cuda", generator=g))):
            P = _gemm.split_rows(X, index, scale)
            ref = X if index is None else torch.gather(X, 1, index.unsqueeze(2).expand(-1, -1, cols))
            if scale is not None:
                ref = scale.unsqueeze(2) * ref
            W = _gemm.split(ref.contiguous())
            assert device_ok(native_lib)
            assert torch.equal(P.to_float(), W.to_float())


@pytest.mark.parametrize("n,other", [(128, 64), (768, 3072), (1200, 768), (672, 100), (1104, 1200), (48, 48)])
@pytest.mark.parametrize("diagreal", [True, False])
def test_operand_dequantized_inside_the_product(native_lib, n, other, diagreal):
    """P G and G P with P taken straight from 4-bit state by the kernel's converter warps: the
    same bytes as dequantizing P into operand planes first (qt_dequantize_planes_f16) and
    multiplying those, for scattered, repeated slots, zero blocks and a tail block included."""
    import qtensor.functional as F
    from optimizers import _gemm
    from optimizers import _engine as E
    dev = "cuda"
    gen = torch.Generator(device=dev).manual_seed(n * 7 + other)
    code = F.create_linear_map(True, 4, 2).to(dev)
    count = 5
    arena = E.QuantArena(n, count, dev, 4, 64, code, 0, diagreal=diagreal)
    X = torch.randn(count, n, n, device=dev, generator=gen) * torch.logspace(-2, 1, count, device=dev).view(-1, 1, 1)
    X[1, :, : min(n, 64)] = 0.0                               # all-zero quantization blocks
    arena.quantize(0, count, X.contiguous())
    slots = [3, 0, 3, 4, 1, 2]
    b = len(slots)
    G_left = torch.randn(b, n, other, device=dev, generator=gen)
    G_right = torch.randn(b, other, n, device=dev, generator=gen)
    planes = arena.dequantize_planes(slots)
    state = arena.operand(slots)
    assert torch.equal(state.exp, planes.exp)
    # P @ G: the 4-bit operand on the A side
    want, _ = _gemm.matmul(planes, _gemm.split(G_left))
    got, _ = _gemm.matmul(state, _gemm.split(G_left))
    assert device_ok(native_lib)
    assert torch.equal(got, want)
    ref = arena.dequantize(0, count)[slots].double() @ G_left.double()
    assert rel(got, ref) < 2e-6
    # G @ P: on the B side, result also handed on as planes
    Gp = _gemm.split(G_right)
    want, wantP = _gemm.matmul(Gp, planes, want_planes=True)
    got, gotP = _gemm.matmul(Gp, state, want_planes=True)
    assert device_ok(native_lib)
    assert torch.equal(got, want) and torch.equal(gotP.to_float(), wantP.to_float())
    ref = G_right.double() @ arena.dequantize(0, count)[slots].double()
    assert rel(got, ref) < 2e-6


@pytest.mark.parametrize("trans_a,trans_b", [(False, True), (False, False), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K,b", [(256, 128, 64, 1), (768, 768, 768, 3), (1200, 1200, 768, 2), (1104, 672, 200, 2),
                                     (200, 72, 50, 5), (1000, 1008, 336, 2), (129, 16, 1200, 1)])
def test_cta_pair_product_equals_single_cta_product(native_lib, trans_a, trans_b, M, N, K, b):
    """The 128 x 192 tile and the cta_group::2 kernel (two CTAs on one 256 x 128 tile, each staging half
    of B) against the 128 x 128 single-CTA kernel on the same planes: same accumulation chains, so the
    results are equal bit for bit - fp32 output, plane output, C operand, ragged rows / columns / k,
    all operand majors."""
    from optimizers import _gemm
    g = torch.Generator(device="cuda").manual_seed(M + 3 * N + 7 * K)
    A = torch.randn((b, K, M) if trans_a else (b, M, K), device="cuda", generator=g)
    B = torch.randn((b, N, K) if trans_b else (b, K, N), device="cuda", generator=g)
    C = torch.randn(b, M, N, device="cuda", generator=g)
    Ap, Bp = _gemm.split(A), _gemm.split(B)
    out = {}
    try:
        for tile in (128, 192, 512):
            native_lib.qt_gemm_force_tile(tile)
            D, P = _gemm.matmul(Ap, Bp, trans_a=trans_a, trans_b=trans_b, alpha=0.75, beta=-1.25, C=C, want_planes=True,
                                out_bound=4.0 * K)
            guard = torch.full((b, M + 3, N + 16), 7.0, device="cuda")
            _gemm.matmul(Ap, Bp, trans_a=trans_a, trans_b=trans_b, out=guard[:, :M, :N])
            assert device_ok(native_lib)
            valid = lambda t: t.view(b, M, P.ld)[:, :, :N].clone()      # the pitch padding is never written
            out[tile] = (D, valid(P.hi), valid(P.lo), guard)
    finally:
        native_lib.qt_gemm_force_tile(-1)
    for other in (192, 512):
        for x, y in zip(out[128], out[other]):
            assert torch.equal(x, y)
    guard = out[512][3]
    assert bool((guard[:, M:, :] == 7.0).all()) and bool((guard[:, :, N:] == 7.0).all())
    ref = 0.75 * ((A.transpose(1, 2) if trans_a else A).double() @ (B.transpose(1, 2) if trans_b else B).double()) - 1.25 * C.double()
    assert rel(out[512][0], ref) < 1e-5, rel(out[512][0], ref)


def test_column_dot_is_accurate_and_independent_of_the_batch(native_lib):
    """Rayleigh quotients diag(V^T (L V)) through qt_column_dot: equal to a float64 evaluation to fp32
    rounding, and a matrix gets the same bits in a batch of 62 as in a batch of 8 (torch's own
    reduction over dim 1 does not: its launch configuration, and with it the order of summation,
    follows the batch size - which made sharded and single-GPU runs drift apart)."""
    from optimizers import _engine as E
    g = torch.Generator(device="cuda").manual_seed(11)
    for n, big, small in ((1200, 62, 8), (768, 20, 1), (100, 7, 2), (50, 3, 1)):
        A = torch.randn(big, n, n, device="cuda", generator=g)
        B = torch.randn(big, n, n, device="cuda", generator=g)
        full = E.column_dot(A, B)
        assert device_ok(native_lib)
        ref = (A.double() * B.double()).sum(dim=1)
        assert float((full.double() - ref).abs().max() / ref.abs().max()) < 1e-6
        part = E.column_dot(A[:small].contiguous(), B[:small].contiguous())
        assert torch.equal(full[:small], part)
