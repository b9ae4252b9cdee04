"""Single kernels through the C ABI against the CPU checker: bit-exact dequantization, the one-token projections, RMS norm, argmax, split attention."""
import ctypes as C

import numpy as np
import pytest
import torch

from dooms_b200 import _lib as L
from dooms_b200.quantize import quantize
from oracle import binding as ob

pytestmark = pytest.mark.gpu

MATRIX_TYPES = [L.F16, L.Q4_0, L.Q5_0, L.Q8_0, L.Q4_K, L.Q6_K]


def random_blocks(dtype, rows, cols, seed):
    """Random block bytes with finite f16 scales: every bit pattern of the quants, scales and mins occurs."""
    if dtype == L.F16:
        g = np.random.default_rng(seed)
        return (g.standard_normal((rows, cols)) * 0.1).astype(np.float16).view(np.uint8).reshape(rows, -1)
    g = np.random.default_rng(seed)
    nb = rows * cols // L.BLOCK_ELEMS[dtype]
    b = g.integers(0, 256, (nb, L.BLOCK_BYTES[dtype]), dtype=np.uint8)
    for off in {L.Q4_0: [0], L.Q5_0: [0], L.Q8_0: [0], L.Q4_K: [0, 2], L.Q6_K: [208]}[dtype]:
        scale = (g.standard_normal(nb) * 0.01).astype(np.float16)
        b[:, off:off + 2] = scale.view(np.uint8).reshape(nb, 2)
    return b.reshape(rows, -1)


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def oracle_matrix(dtype, blocks, rows, cols):
    return np.stack([ob.dequantize(dtype, blocks[r], cols) for r in range(rows)])


@pytest.mark.parametrize("dtype", MATRIX_TYPES)
@pytest.mark.parametrize("shape", [(3, 256), (17, 1024), (1, 512), (64, 4864 if True else 0)])
def test_dequantize_is_bit_exact(dtype, shape):
    rows, cols = shape
    if cols % L.BLOCK_ELEMS[dtype]:
        cols = cols // 256 * 256
    blocks = random_blocks(dtype, rows, cols, 7)
    want = oracle_matrix(dtype, blocks, rows, cols)
    d_blocks, d_out = dev(blocks), torch.empty(rows, cols, dtype=torch.float32, device="cuda")
    L.check(L.lib().dooms_cuda_dequantize(dtype, d_blocks.data_ptr(), rows, cols, d_out.data_ptr(), None))
    torch.cuda.synchronize()
    got = d_out.cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("dtype", MATRIX_TYPES)
def test_dequantize_of_quantized_normal_weights_is_bit_exact(dtype):
    x = torch.randn(32, 2048, generator=torch.Generator().manual_seed(3)) * 0.02
    blocks = quantize(dtype, x).numpy()
    want = oracle_matrix(dtype, blocks, 32, 2048)
    d_blocks, d_out = dev(blocks), torch.empty(32, 2048, dtype=torch.float32, device="cuda")
    L.check(L.lib().dooms_cuda_dequantize(dtype, d_blocks.data_ptr(), 32, 2048, d_out.data_ptr(), None))
    torch.cuda.synchronize()
    assert np.array_equal(d_out.cpu().numpy().view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("dtype", MATRIX_TYPES)
@pytest.mark.parametrize("shape", [(1152, 896), (896, 4864), (50, 256), (7, 2304), (300, 4096), (64, 14336)])
def test_matvec_matches_the_oracle(dtype, shape):
    rows, cols = shape
    if cols % L.BLOCK_ELEMS[dtype]:
        pytest.skip("rows are not whole blocks of this type")
    blocks = random_blocks(dtype, rows, cols, 11)
    g = np.random.default_rng(5)
    x = g.standard_normal(cols).astype(np.float32)
    bias = g.standard_normal(rows).astype(np.float32)
    y0 = g.standard_normal(rows).astype(np.float32)
    w = oracle_matrix(dtype, blocks, rows, cols).astype(np.float64)
    base = w @ x.astype(np.float64)
    scale = np.abs(w).astype(np.float64) @ np.abs(x).astype(np.float64)          # size of the terms, for a per-row bound
    d_w, d_x, d_b = dev(blocks), dev(x), dev(bias)
    for flags, want in ((0, base), (4, base + bias), (2, base + y0), (6, base + bias + y0)):
        d_y = dev(y0.copy())
        L.check(L.lib().dooms_cuda_matvec(dtype, d_w.data_ptr(), d_x.data_ptr(), d_y.data_ptr(), d_b.data_ptr(), rows, cols, flags, None))
        torch.cuda.synchronize()
        got = d_y.cpu().numpy().astype(np.float64)
        assert np.all(np.abs(got - want) <= 2e-6 * scale + 1e-6 * np.abs(want) + 1e-30), (flags, np.abs(got - want).max())


@pytest.mark.parametrize("dtype", MATRIX_TYPES)
def test_gate_up_matches_the_oracle(dtype):
    rows, cols = 4864, 1024
    bg, bu = random_blocks(dtype, rows, cols, 1), random_blocks(dtype, rows, cols, 2)
    x = np.random.default_rng(3).standard_normal(cols).astype(np.float32)
    g = oracle_matrix(dtype, bg, rows, cols).astype(np.float64) @ x
    u = oracle_matrix(dtype, bu, rows, cols).astype(np.float64) @ x
    want = g / (1 + np.exp(-g)) * u
    d_h = torch.empty(rows, dtype=torch.float32, device="cuda")
    d_g, d_u, d_x = dev(bg), dev(bu), dev(x)          # named: the device buffers must outlive the launch
    L.check(L.lib().dooms_cuda_gate_up(dtype, d_g.data_ptr(), d_u.data_ptr(), d_x.data_ptr(), d_h.data_ptr(), rows, cols, None))
    torch.cuda.synchronize()
    got = d_h.cpu().numpy()
    assert np.sqrt(((got - want) ** 2).sum() / (want ** 2).sum()) < 1e-5


@pytest.mark.parametrize("dtype,shape", [(L.Q4_0, (300, 4096)), (L.Q4_0, (1152, 896)), (L.Q4_K, (64, 14336)), (L.Q4_0, (4864, 1024))])
def test_projections_on_an_input_that_is_already_split_give_the_same_bits(dtype, shape):
    """The integer tensor-core kernel on the split a producer kernel would leave (dooms_cuda_split_input) against the same kernel splitting the f32 input
    itself: identical results, plain and gate / up."""
    rows, cols = shape
    lib = L.lib()
    bw, bu = random_blocks(dtype, rows, cols, 21), random_blocks(dtype, rows, cols, 22)
    x = np.random.default_rng(9).standard_normal(cols).astype(np.float32)
    d_w, d_u, d_x = dev(bw), dev(bu), dev(x)
    d_split = torch.empty(lib.dooms_cuda_split_input_bytes(cols), dtype=torch.uint8, device="cuda")
    L.check(lib.dooms_cuda_split_input(d_x.data_ptr(), cols, d_split.data_ptr(), None))
    a, b = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
    L.check(lib.dooms_cuda_matvec(dtype, d_w.data_ptr(), d_x.data_ptr(), a.data_ptr(), None, rows, cols, 0, None))
    L.check(lib.dooms_cuda_matvec_split(dtype, d_w.data_ptr(), None, d_split.data_ptr(), b.data_ptr(), None, rows, cols, 0, None))
    torch.cuda.synchronize()
    assert torch.equal(a, b)
    L.check(lib.dooms_cuda_gate_up(dtype, d_w.data_ptr(), d_u.data_ptr(), d_x.data_ptr(), a.data_ptr(), rows, cols, None))
    L.check(lib.dooms_cuda_matvec_split(dtype, d_w.data_ptr(), d_u.data_ptr(), d_split.data_ptr(), b.data_ptr(), None, rows, cols, 0, None))
    torch.cuda.synchronize()
    assert torch.equal(a, b)
    assert lib.dooms_cuda_matvec_split(L.Q8_0, d_w.data_ptr(), None, d_split.data_ptr(), b.data_ptr(), None, rows, cols, 0, None) == L.UNSUPPORTED


def test_rms_norm_matches_the_oracle():
    g = np.random.default_rng(0)
    x = g.standard_normal((5, 896)).astype(np.float32) * 3
    gamma = g.uniform(0.7, 1.3, 896).astype(np.float32)
    xd = x.astype(np.float64)
    want = xd / np.sqrt((xd ** 2).mean(axis=1, keepdims=True) + 1e-6) * gamma
    d_out = torch.empty(5, 896, dtype=torch.float32, device="cuda")
    d_x, d_g = dev(x), dev(gamma)
    L.check(L.lib().dooms_cuda_rms_norm(d_x.data_ptr(), d_g.data_ptr(), d_out.data_ptr(), 5, 896, 1e-6, None))
    torch.cuda.synchronize()
    assert np.abs(d_out.cpu().numpy() - want).max() < 1e-5


def gpu_argmax(v):
    d_out = torch.zeros(1, dtype=torch.int32, device="cuda")
    d_v = dev(v)
    L.check(L.lib().dooms_cuda_argmax(d_v.data_ptr(), v.size, d_out.data_ptr(), None))
    torch.cuda.synchronize()
    return int(d_out.item())


def test_argmax_first_index_ties_and_nan():
    """The reference's argmax cases (tests/unit/test_argmax.cpp:23-74): first index on ties, NaN never wins, a vocabulary-sized vector."""
    assert gpu_argmax(np.array([1, 3, 3, 2], dtype=np.float32)) == 1
    assert gpu_argmax(np.array([np.nan, 1, 2], dtype=np.float32)) == 2
    assert gpu_argmax(np.array([np.nan, np.nan], dtype=np.float32)) == 0
    assert gpu_argmax(np.array([-np.inf, -np.inf], dtype=np.float32)) == 0
    assert gpu_argmax(np.array([5], dtype=np.float32)) == 0
    g = np.random.default_rng(1)
    for n in (151936, 128256, 4097, 31):
        v = g.standard_normal(n).astype(np.float32)
        assert gpu_argmax(v) == ob.argmax(v) == int(np.argmax(v))
        v[n // 3] = v[n - 1] = v.max() + 1          # a tie far apart: the first wins
        assert gpu_argmax(v) == n // 3
        v[5] = np.nan
        assert gpu_argmax(v) == n // 3
    zeros = np.zeros(151936, dtype=np.float32)
    assert gpu_argmax(zeros) == 0


@pytest.mark.parametrize("n_head,n_head_kv,head_dim,n_keys", [(14, 2, 64, 1), (14, 2, 64, 700), (32, 8, 128, 2304), (4, 2, 16, 45), (40, 8, 128, 8448),
                                                               (6, 6, 64, 130), (16, 2, 128, 64), (4, 2, 64, 65), (24, 2, 64, 300)])
def test_split_attention_matches_the_oracle(n_head, n_head_kv, head_dim, n_keys):
    g = np.random.default_rng(n_keys)
    q = g.standard_normal((n_head, head_dim)).astype(np.float32)
    kc = g.standard_normal((n_keys, n_head_kv * head_dim)).astype(np.float16)
    vc = g.standard_normal((n_keys, n_head_kv * head_dim)).astype(np.float16)
    want = np.empty((n_head, head_dim))
    for h in range(n_head):
        kv = h // (n_head // n_head_kv)
        k = kc[:, kv * head_dim:(kv + 1) * head_dim].astype(np.float64)
        v = vc[:, kv * head_dim:(kv + 1) * head_dim].astype(np.float64)
        s = k @ q[h].astype(np.float64) / np.sqrt(head_dim)
        p = np.exp(s - s.max())
        want[h] = (p / p.sum()) @ v
    nbytes = L.lib().dooms_cuda_attention_scratch_bytes(n_head, head_dim, n_keys)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    d_out = torch.empty(n_head, head_dim, dtype=torch.float32, device="cuda")
    d_q, d_k, d_v = dev(q), dev(kc), dev(vc)
    L.check(L.lib().dooms_cuda_attention_decode(d_q.data_ptr(), d_k.data_ptr(), d_v.data_ptr(), d_out.data_ptr(), scratch.data_ptr(), n_head,
                                                n_head_kv, head_dim, n_keys, None))
    torch.cuda.synchronize()
    assert np.abs(d_out.cpu().numpy() - want).max() < 2e-5


def test_kernel_entry_points_reject_bad_arguments():
    lib = L.lib()
    assert lib.dooms_cuda_dequantize(L.F32, 1, 1, 32, 1, None) == L.UNSUPPORTED
    assert lib.dooms_cuda_dequantize(L.Q4_0, None, 1, 32, 1, None) == L.INVALID_ARGUMENT
    assert lib.dooms_cuda_dequantize(L.Q4_K, 1, 1, 32, 1, None) == L.INVALID_ARGUMENT          # not a whole block
    assert lib.dooms_cuda_matvec(L.Q4_0, 1, 1, 1, None, 4, 64, 4, None) == L.INVALID_ARGUMENT  # bias flag without a bias
    assert lib.dooms_cuda_argmax(None, 5, None, None) == L.INVALID_ARGUMENT
    assert lib.dooms_cuda_attention_decode(1, 1, 1, 1, 1, 4, 2, 24, 8, None) == L.UNSUPPORTED


@pytest.mark.parametrize("dtype", MATRIX_TYPES)
@pytest.mark.parametrize("shape", [(45, 300, 256), (130, 128, 512), (1, 129, 64), (257, 256, 1024), (600, 200, 512), (2000, 2500, 1024)])
@pytest.mark.parametrize("gate", [False, True])
def test_tensor_core_matmul_matches_the_oracle(dtype, shape, gate):
    """The tcgen05 prefill GEMM against float64 products of the checker's dequantized weights rounded to f16 (the operand rounding of the reference's
    tiles, src/backend/metal/llama_kernels.h:186-199); tokens and rows that are no multiple of the 128-wide tiles. From 128 tokens on the entry point
    dequantizes the matrix to f16 rows first and feeds both operands by TMA (except q4_0 / q4_K gate / up, which stay fused). The last shape is 160
    tiles: more than one wave of blocks, so its one-matrix form runs as blocks of 256 weight rows and its fused gate / up form deals the reduction of
    the tiles left over after the last full wave over the idle SMs."""
    tokens, rows, cols = shape
    if cols % L.BLOCK_ELEMS[dtype]:
        pytest.skip("rows are not whole blocks of this type")
    g = np.random.default_rng(3)
    bw, bw2 = random_blocks(dtype, rows, cols, 21), random_blocks(dtype, rows, cols, 22)
    x16 = g.standard_normal((tokens, cols)).astype(np.float16)
    bias = g.standard_normal(rows).astype(np.float32)
    y0 = g.standard_normal((tokens, rows)).astype(np.float32)
    w = oracle_matrix(dtype, bw, rows, cols).astype(np.float16).astype(np.float64)
    base = x16.astype(np.float64) @ w.T
    d_w, d_w2, d_x, d_b = dev(bw), dev(bw2), dev(x16), dev(bias)
    if gate:
        u = x16.astype(np.float64) @ oracle_matrix(dtype, bw2, rows, cols).astype(np.float16).astype(np.float64).T
        cases = [(0, base / (1 + np.exp(-base)) * u)]
    else:
        cases = [(0, base), (4, base + bias), (2, base + y0), (6, base + bias + y0)]
    for flags, want in cases:
        d_y = dev(y0.copy())
        L.check(L.lib().dooms_cuda_matmul(dtype, d_w.data_ptr(), d_w2.data_ptr() if gate else None, d_x.data_ptr(), d_y.data_ptr(), d_b.data_ptr(), tokens,
                                          rows, cols, flags, None))
        flag = C.c_int32(-1)
        L.check(L.lib().dooms_cuda_kernel_status(None, C.byref(flag)))       # waits for the stream; no bounded wait gave up
        assert flag.value == 0
        got = d_y.cpu().numpy().astype(np.float64)
        assert np.isfinite(got).all()
        assert np.sqrt(((got - want) ** 2).sum() / (want ** 2).sum()) < 2e-5, flags
