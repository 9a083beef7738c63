"""GPU parity of the blockwise quantizer: CUDA kernels (through the C ABI) vs the CPU oracle
and vs the committed outputs of the reference.  Bit-exact: codes, absmax, diag and the
dequantized matrix (bit patterns, including the sign of zero)."""
import ctypes as ct

import numpy as np
import pytest
import torch

from helpers import bits_equal, case_ids, load_quant_cases, spd_logspectrum
from oracle import qoracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def F(native_lib):
    import qtensor.functional as F
    assert F.lib is not None, "native library must be loaded for GPU tests"
    return F


def t_bf16_bits(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def from_bf16_bits(a, device):
    return torch.from_numpy(a.view(np.int16).copy()).to(device).view(torch.bfloat16)


def run_gpu(F, A_np, code_np, n, bs, bits, diagreal, in_bf16=False, out_bf16=False):
    dev = "cuda:0"
    A = from_bf16_bits(A_np, dev).reshape(n, n) if in_bf16 else torch.from_numpy(np.ascontiguousarray(A_np, dtype=np.float32)).to(dev).reshape(n, n)
    code = torch.from_numpy(code_np).to(dev)
    outdtype = torch.bfloat16 if out_bf16 else torch.float32
    if diagreal:
        q, am, dg = F.quantize_blockwise_diagreal(A, code, n, blocksize=bs, bits=bits)
        d = F.dequantize_blockwise_diagreal(q, code, n, am, dg, outdtype=outdtype, blocksize=bs, bits=bits)
        dg = dg.cpu().numpy()
    else:
        q, am = F.quantize_blockwise(A, code, n, blocksize=bs, bits=bits)
        d = F.dequantize_blockwise(q, code, n, am, outdtype=outdtype, blocksize=bs, bits=bits)
        dg = None
    assert d is not None and d.shape == (n, n)
    torch.cuda.synchronize()
    d = t_bf16_bits(d) if out_bf16 else d.cpu().numpy()
    return q.cpu().numpy(), am.cpu().numpy(), dg, d


def check_against_oracle(F, A_np, code_np, n, bs, bits, diagreal, in_bf16=False, out_bf16=False):
    q, am, dg, d = run_gpu(F, A_np, code_np, n, bs, bits, diagreal, in_bf16, out_bf16)
    ref = qoracle.quantize(A_np, code_np, n, bs, bits, store_diag=diagreal)
    assert bits_equal(q, ref[0]), f"codes differ in {(q != ref[0]).sum()} bytes"
    assert bits_equal(am, ref[1])
    if diagreal:
        assert bits_equal(dg, ref[2])
    rd = qoracle.dequantize(ref[0], code_np, n, ref[1], bs, bits, diag=ref[2] if diagreal else None, out_bf16=out_bf16)
    assert bits_equal(d, rd)


@pytest.mark.parametrize("name", case_ids())
def test_gpu_matches_reference_fixture(F, name):
    blob, index = load_quant_cases()
    c = next(i for i in index if i["name"] == name)
    code = blob["code." + c["code"]]
    q, am, dg, d = run_gpu(F, blob[name + ".A"], code, c["order"], c["blocksize"], c["bits"], c["diagreal"],
                           c["in_bf16"], c["out_bf16"])
    assert bits_equal(q, blob[name + ".packed"])
    assert bits_equal(am, blob[name + ".absmax"])
    if c["diagreal"]:
        assert bits_equal(dg, blob[name + ".diag"])
    assert bits_equal(d, blob[name + ".deq"])


@pytest.mark.parametrize("diagreal", [False, True])
def test_every_small_order(F, diagreal):
    """orders 1..130: odd orders, tails, rows that straddle bytes."""
    code = qoracle.linear_map(True, 4, 2)
    rng = np.random.default_rng(5)
    for n in range(1, 131):
        A = (rng.standard_normal((n, n)) * 10.0 ** rng.integers(-6, 3)).astype(np.float32)
        check_against_oracle(F, A, code, n, 64, 4, diagreal)


@pytest.mark.parametrize("bs", [64, 128, 256, 512, 1024, 2048])
@pytest.mark.parametrize("bits", [4, 8])
def test_block_sizes_and_bits(F, bs, bits):
    code = qoracle.linear_map(True, bits, 2)
    rng = np.random.default_rng(bs + bits)
    for n in (96, 264, 1000, 2100):
        A = (rng.standard_normal((n, n)) * np.logspace(-5, 1, n)[None, :]).astype(np.float32)
        A[n // 2, :] = 0.0
        for diagreal in (False, True):
            check_against_oracle(F, A, code, n, bs, bits, diagreal)


@pytest.mark.parametrize("n", [64, 100, 336, 672, 768, 1000, 1008, 1104, 1152, 1200])
def test_model_orders_fp32_and_bf16(F, n):
    """Preconditioner orders that occur in the ResNet-34 / Swin-T / ViT-B/32 workloads."""
    code = qoracle.linear_map(True, 4, 2)
    rng = np.random.default_rng(n)
    A = rng.standard_normal((n, n)).astype(np.float32)
    A[:, : n // 3] *= 1e-4
    check_against_oracle(F, A, code, n, 64, 4, False)
    check_against_oracle(F, A, code, n, 64, 4, True)
    A16 = (torch.from_numpy(A).bfloat16().view(torch.int16).numpy().view(np.uint16))
    check_against_oracle(F, A16, code, n, 64, 4, True, in_bf16=True, out_bf16=True)
    eye = np.eye(n, dtype=np.float32)
    check_against_oracle(F, eye, code, n, 64, 4, False)
    check_against_oracle(F, eye * np.float32(1e-6), code, n, 64, 4, True)


def test_other_codebooks(F):
    rng = np.random.default_rng(11)
    A = rng.standard_normal((200, 200)).astype(np.float32)
    check_against_oracle(F, A, qoracle.dynamic_map(True, 4, 1), 200, 64, 4, False)
    check_against_oracle(F, A, qoracle.dynamic_map(True, 8, 1), 200, 64, 8, True)
    shuffled = qoracle.linear_map(True, 4, 2)[rng.permutation(16)].copy()
    check_against_oracle(F, A, shuffled, 200, 64, 4, True)
    uniform = np.linspace(-1, 1, 16).astype(np.float32)       # no exact zero, threshold at 0
    check_against_oracle(F, A, uniform, 200, 64, 4, False)


def test_near_threshold_values(F):
    """Inputs placed within a few ulps of every decision threshold of the codebook."""
    code = qoracle.linear_map(True, 4, 2)
    mids = ((code[:-1].astype(np.float64) + code[1:]) / 2).astype(np.float32)
    vals = []
    for m in mids:
        v = m
        for _ in range(6):
            v = np.nextafter(v, np.float32(-2))
        for _ in range(13):
            vals.append(v)
            v = np.nextafter(v, np.float32(2))
    vals = np.array(vals, dtype=np.float32)
    n = 256
    rng = np.random.default_rng(3)
    A = rng.choice(vals, size=(n, n)).astype(np.float32)
    A[:, 0::64] = 1.0                                         # absmax 1 in every block
    check_against_oracle(F, A, code, n, 64, 4, False)
    scale = rng.uniform(0.5, 3.0, size=(n, 1)).astype(np.float32)
    check_against_oracle(F, (A * scale).astype(np.float32), code, n, 64, 4, False)


def test_config1_spd_1024(F):
    """The 1024 x 1024 SPD matrix with log-uniform spectrum, block 64, 4-bit, plain and diagreal."""
    A = spd_logspectrum(1024, 0).numpy()
    code = qoracle.linear_map(True, 4, 2)
    check_against_oracle(F, A, code, 1024, 64, 4, False)
    check_against_oracle(F, A, code, 1024, 64, 4, True)


def test_large_and_batched_properties(F, native_lib):
    """Full-size checks through size-independent properties: a strided batch equals the
    per-matrix calls, and quantize(dequantize(codes)) reproduces codes and scales."""
    lib = native_lib
    dev = "cuda:0"
    n, count, bs = 4096, 6, 64
    g = torch.Generator(device=dev).manual_seed(9)
    A = torch.randn(count, n, n, device=dev, generator=g) / n ** 0.5
    code = torch.from_numpy(qoracle.linear_map(True, 4, 2)).to(dev)
    nb = (n + bs - 1) // bs
    packed = torch.empty(count, n * n // 2, dtype=torch.uint8, device=dev)
    absmax = torch.empty(count, n * nb, device=dev)
    diag = torch.empty(count, n, device=dev)
    stream = ct.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: ct.c_void_p(t.data_ptr())
    rc = lib.qt_quantize_blockwise(p(A), 0, n * n, p(code), n, count, p(absmax), n * nb, p(diag), n,
                                   p(packed), n * n // 2, bs, 4, stream)
    assert rc == 0
    out = torch.empty(count, n, n, device=dev)
    rc = lib.qt_dequantize_blockwise(p(packed), n * n // 2, p(code), n, count, p(absmax), n * nb, p(diag), n,
                                     p(out), 0, n * n, bs, 4, stream)
    assert rc == 0
    for m in (0, count - 1):
        q1, a1, d1 = F.quantize_blockwise_diagreal(A[m], code, n, blocksize=bs, bits=4)
        assert torch.equal(q1, packed[m]) and torch.equal(a1, absmax[m]) and torch.equal(d1, diag[m])
        o1 = F.dequantize_blockwise_diagreal(q1, code, n, a1, d1, blocksize=bs, bits=4)
        assert torch.equal(o1.view(torch.int32), out[m].view(torch.int32))
    # one matrix against the CPU oracle at full size
    ref = qoracle.quantize(A[1].cpu().numpy(), code.cpu().numpy(), n, bs, 4, store_diag=True)
    assert bits_equal(packed[1].cpu().numpy(), ref[0]) and bits_equal(absmax[1].cpu().numpy(), ref[1])
    # idempotence
    packed2 = torch.empty_like(packed)
    absmax2 = torch.empty_like(absmax)
    diag2 = torch.empty_like(diag)
    rc = lib.qt_quantize_blockwise(p(out), 0, n * n, p(code), n, count, p(absmax2), n * nb, p(diag2), n,
                                   p(packed2), n * n // 2, bs, 4, stream)
    assert rc == 0
    assert torch.equal(packed2, packed) and torch.equal(absmax2, absmax) and torch.equal(diag2, diag)
    # the diagonal survives in fp32
    assert torch.equal(torch.diagonal(out, dim1=1, dim2=2), torch.diagonal(A, dim1=1, dim2=2))


def test_legacy_symbols_drop_in(F, native_lib):
    """The sixteen symbols the reference's ctypes code binds, called the way it calls them
    (raw pointers, c_int32 order/blocksize, no argtypes), on the legacy default stream."""
    lib = native_lib
    dev = "cuda:0"
    n, bs = 200, 64
    rng = np.random.default_rng(21)
    A_np = rng.standard_normal((n, n)).astype(np.float32)
    P = lambda t: ct.c_void_p(t.data_ptr())
    lib.qt_set_stream(ct.c_void_p(0))
    for bits in (4, 8):
        code_np = qoracle.linear_map(True, bits, 2)
        code = torch.from_numpy(code_np).to(dev)
        for dt in ("fp32", "bf16"):
            A = torch.from_numpy(A_np).to(dev)
            if dt == "bf16":
                A = A.bfloat16()
            A_host = t_bf16_bits(A) if dt == "bf16" else A_np
            for diagreal in (False, True):
                kind = "diagreal_" if diagreal else ""
                nb = (n + bs - 1) // bs
                absmax = torch.empty(n * nb, device=dev)
                diag = torch.empty(n, device=dev)
                out = torch.empty((n * n * bits + 7) // 8, dtype=torch.uint8, device=dev)
                deq = torch.empty(n, n, device=dev, dtype=A.dtype)
                torch.cuda.synchronize()
                qf = getattr(lib, f"cquantize_blockwise_{kind}{bits}bit_{dt}")
                df = getattr(lib, f"cdequantize_blockwise_{kind}{bits}bit_{dt}")
                if diagreal:
                    qf(P(A), P(code), ct.c_int32(n), P(absmax), P(diag), P(out), ct.c_int32(bs))
                    df(P(out), P(code), ct.c_int32(n), P(absmax), P(diag), P(deq), ct.c_int32(bs))
                else:
                    qf(P(A), P(code), ct.c_int32(n), P(absmax), P(out), ct.c_int32(bs))
                    df(P(out), P(code), ct.c_int32(n), P(absmax), P(deq), ct.c_int32(bs))
                assert lib.qt_last_error() == 0
                torch.cuda.synchronize()
                ref = qoracle.quantize(A_host, code_np, n, bs, bits, store_diag=diagreal)
                assert bits_equal(out.cpu().numpy(), ref[0])
                assert bits_equal(absmax.cpu().numpy(), ref[1])
                rd = qoracle.dequantize(ref[0], code_np, n, ref[1], bs, bits, diag=ref[2] if diagreal else None,
                                        out_bf16=(dt == "bf16"))
                got = t_bf16_bits(deq) if dt == "bf16" else deq.cpu().numpy()
                assert bits_equal(got, rd)


def test_output_canaries_untouched(F):
    """Kernels write exactly ceil(n*n/2) bytes, n*nb scales and n*n values: guard words survive."""
    dev = "cuda:0"
    code = torch.from_numpy(qoracle.linear_map(True, 4, 2)).to(dev)
    for n in (65, 100, 1000):
        nb = (n + 63) // 64
        nbytes = (n * n + 1) // 2
        A = torch.randn(n, n, device=dev)
        out = torch.full((nbytes + 64,), 0xAB, dtype=torch.uint8, device=dev)
        absmax = torch.full((n * nb + 16,), -7.0, device=dev)
        F.quantize_blockwise(A, code, n, absmax=absmax[: n * nb], out=out[:nbytes], blocksize=64, bits=4)
        assert bool((out[nbytes:] == 0xAB).all()) and bool((absmax[n * nb:] == -7.0).all())
        deq = torch.full((n * n + 32,), -3.0, device=dev)
        F.dequantize_blockwise(out[:nbytes], code, n, absmax[: n * nb], out=deq[: n * n].view(n, n), blocksize=64, bits=4)
        assert bool((deq[n * n:] == -3.0).all())


def test_fast_division_is_bit_identical_to_ieee_division(native_lib):
    """2^31 pseudo-random (x, absmax) pairs: reciprocal + two FMA corrections == x / absmax, bit for bit."""
    counter = torch.zeros(1, dtype=torch.int64, device="cuda:0")
    for seed in (1, 2):
        rc = native_lib.qt_selftest_division(seed, 1 << 30, ct.c_void_p(counter.data_ptr()),
                                             ct.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert rc == 0
    torch.cuda.synchronize()
    assert int(counter.item()) == 0


@pytest.mark.parametrize("n,bits,diagreal", [(768, 4, True), (1200, 4, True), (72, 4, False), (256, 8, True), (1000, 4, True)])
def test_dequantize_to_planes_equals_dequantize_then_split(native_lib, n, bits, diagreal):
    """qt_dequantize_planes (with a slot gather) writes exactly the bf16 hi/lo planes that
    dequantize -> split produce, for scattered and repeated slots."""
    import ctypes as ct
    import qtensor.functional as F
    from optimizers import _engine as E, _gemm
    dev = "cuda"
    code = F.create_linear_map(True, bits, 2).to(dev)
    count = 7
    arena = E.QuantArena(n, count, dev, bits, 64, code, 4096, diagreal=diagreal)
    g = torch.Generator(device=dev).manual_seed(n + bits)
    X = torch.randn(count, n, n, device=dev, generator=g) * torch.logspace(-4, 2, count, device=dev)[:, None, None]
    X[2].zero_()
    arena.quantize(0, count, X)
    slots = [5, 0, 2, 2, 6]
    P = arena.dequantize_planes(slots)
    full = arena.dequantize(0, count)
    want = _gemm.split(full[slots].contiguous())
    torch.cuda.synchronize()
    assert native_lib.qt_last_error() == 0
    k = (n - 1) * P.ld + n
    hi, lo = P.hi.view(len(slots), n, P.ld)[:, :, :n], P.lo.view(len(slots), n, P.ld)[:, :, :n]
    whi, wlo = want.hi.view(len(slots), n, want.ld)[:, :, :n], want.lo.view(len(slots), n, want.ld)[:, :, :n]
    assert torch.equal(hi.view(torch.int16), whi.view(torch.int16))
    assert torch.equal(lo.view(torch.int16), wlo.view(torch.int16))
