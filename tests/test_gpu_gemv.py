"""GPU parity of the Q4_K x Q8_1 path against the CPU oracle: dequant and integer block dots bit-exact,
GEMV bit-exact against the canonical-order oracle and within 1e-3 of the plain restatement."""
import numpy as np
import pytest

from bunker_b200 import ops, synth
from bunker_b200 import runtime as R
from oracle import oracle as O
from tests.util import assert_same_bits, dev, rel_err

pytestmark = pytest.mark.gpu


def test_dequant_bit_exact(bk):
    N, K = 96, 1024
    W = synth.q4k_weights(np.random.default_rng(1), N, K)
    dW, out = dev(W), R.DeviceBuffer(N * K * 4)
    ops.dequant_q4k(dW.ptr, N, K, out.ptr)
    assert_same_bits(out.download(np.float32, (N, K)), O.q4k_dequant(W, N, K), "dequant")


def test_dequant_denormal_and_extreme_headers(bk):
    # d/dmin below the smallest normal half, scale bytes of all ones / all zeros
    N, K = 4, 512
    W = synth.q4k_weights(np.random.default_rng(2), N, K).reshape(N, K // 256, 144)
    W[0, :, 0:4] = np.array([1e-6, 3e-7], np.float16).view(np.uint8)
    W[1, :, 4:16] = 0xFF
    W[2, :, 4:16] = 0
    W[3, :, 16:] = 0xFF
    W = W.reshape(N, -1)
    dW, out = dev(W), R.DeviceBuffer(N * K * 4)
    ops.dequant_q4k(dW.ptr, N, K, out.ptr)
    assert_same_bits(out.download(np.float32, (N, K)), O.q4k_dequant(W, N, K), "dequant edge")


@pytest.mark.parametrize("bf16", [False, True])
def test_quant_q8_1_bit_exact(bk, bf16):
    B, K = 3, 2048
    x = np.random.default_rng(3).normal(0, 1, (B, K)).astype(np.float32)
    x[0, :32] = 0.0          # all-zero block
    x[1, 32:64] = 1e-30      # scale below half range
    x[2, 64] = 3e4           # large magnitude
    if bf16:
        xb = synth.f32_to_bf16(x)
        want = O.q8_1_quantize_bf16(xb)
        dx = dev(xb)
    else:
        want = O.q8_1_quantize(x)
        dx = dev(x)
    out = R.DeviceBuffer(B * K // 32 * 36)
    ops.quant_q8_1(dx.ptr, K, B, out.ptr, bf16=bf16)
    assert_same_bits(out.download(np.uint8, (B, K // 32, 36)), want, "q8_1 blocks")


def test_block_dots_bit_exact(bk):
    N, K = 64, 2048
    W, x = synth.gemv_case(N, K, 1)
    xq = O.q8_1_quantize(x)
    dW, dx = dev(W), dev(xq)
    di, dq = R.DeviceBuffer(N * K // 32 * 4), R.DeviceBuffer(N * K // 32 * 4)
    ops.block_dots(dW.ptr, N, K, dx.ptr, di.ptr, dq.ptr)
    gi, gq = di.download(np.int32, (N, K // 32)), dq.download(np.int32, (N, K // 32))
    for n in range(N):
        wi, wq = O.block_dots(W[n], xq[0], K)
        assert np.array_equal(gi[n], wi) and np.array_equal(gq[n], wq), f"row {n}"


def test_gemv_config0(bk):
    """configs[0]: 4096x4096 Q4_K, x f32 N(0,1) -> Q8_1, y f32."""
    N, K = 4096, 4096
    W, x = synth.gemv_case(N, K, 1)
    dW, dx = dev(W), dev(x)
    dxq, dy = R.DeviceBuffer(K // 32 * 36), R.DeviceBuffer(N * 4)
    ops.quant_q8_1(dx.ptr, K, 1, dxq.ptr)
    ops.gemv_simple(dW.ptr, N, K, dxq.ptr, 1, dy.ptr)
    y = dy.download(np.float32, (1, N))
    xq = O.q8_1_quantize(x)
    assert_same_bits(dxq.download(np.uint8, (1, K // 32, 36)), xq, "xq")
    assert_same_bits(y, O.gemv_q4k_q8(W, N, K, xq), "gemv canonical")
    assert rel_err(y, O.gemv_q4k_q8_plain(W, N, K, xq)) < 1e-3


@pytest.mark.parametrize("B", [1, 2, 3, 4, 5, 6, 7, 8])
@pytest.mark.parametrize("K", [256, 2048, 6144])
def test_gemv_batches_and_tails(bk, B, K):
    N = 131  # odd: exercises the unpaired last row
    W, x = synth.gemv_case(N, K, B, config_id=10 + B)
    xq = O.q8_1_quantize(x)
    dW, dxq, dy = dev(W), dev(xq), R.DeviceBuffer(B * N * 4)
    ops.gemv_simple(dW.ptr, N, K, dxq.ptr, B, dy.ptr)
    assert_same_bits(dy.download(np.float32, (B, N)), O.gemv_q4k_q8(W, N, K, xq), f"gemv B={B} K={K}")


@pytest.mark.parametrize("B,K", [(2, 2048), (3, 2048), (8, 2048), (5, 4096), (8, 6144), (8, 5120)])
def test_gemv_staged_activation(bk, B, K):
    """Batch 3..8: the activation arrives as the staged image written by the norm+quantise launch; SwiGLU and
    plain segments; same bits as the oracle's RMSNorm -> Q8_1 -> GEMV."""
    N = 300
    rng = np.random.default_rng(90 + B + K)
    Wg, Wu = synth.q4k_weights(rng, N, K), synth.q4k_weights(rng, N, K)
    x, nw = synth.normal_bf16(rng, (B, K)), synth.normal_bf16(rng, (K,), 0.02)
    xq = O.q8_1_quantize_bf16(O.rmsnorm(x, nw))
    dx, dnw, dWg, dWu = dev(x), dev(nw), dev(Wg), dev(Wu)
    img = R.DeviceBuffer.zeros(ops.staged_bytes(K, B))
    ops.rmsnorm_quant_q8_1(dx.ptr, dnw.ptr, K, B, img.ptr, layout=R.BK_Q8_STAGED)
    act, y = R.DeviceBuffer(B * N * 2), R.DeviceBuffer(B * N * 4)
    ops.gemv(img.ptr, K, B, [ops.gemv_seg(dWg.ptr, N, act.ptr, R.BK_EPI_SWIGLU, W2=dWu.ptr)], prologue=R.BK_PRO_STAGED)
    ops.gemv(img.ptr, K, B, [ops.gemv_seg(dWg.ptr, N, y.ptr, R.BK_EPI_F32)], prologue=R.BK_PRO_STAGED)
    g, u = O.gemv_q4k_q8(Wg, N, K, xq), O.gemv_q4k_q8(Wu, N, K, xq)
    assert_same_bits(y.download(np.float32, (B, N)), g, "f32 segment from a staged activation")
    assert_same_bits(act.download(np.uint16, (B, N)), O.swiglu(g, u), "SwiGLU segment from a staged activation")
    with pytest.raises(R.BunkerCudaError):   # batch 1 has no staged path
        ops.gemv(img.ptr, K, 1, [ops.gemv_seg(dWg.ptr, N, y.ptr, R.BK_EPI_F32)], prologue=R.BK_PRO_STAGED)


@pytest.mark.parametrize("B", [9, 16, 20, 32])
def test_gemv_more_than_eight_columns(bk, B):
    """Batch 9..32 runs as groups of 8 columns (a last group of one column takes the batch-1 kernel): Q8_1 blocks in,
    bf16 rows in with the fused norm, and -- unless a group of one is left over -- the grouped staged image."""
    K, N = 2048, 150
    rng = np.random.default_rng(200 + B)
    W = synth.q4k_weights(rng, N, K)
    x, nw = synth.normal_bf16(rng, (B, K)), synth.normal_bf16(rng, (K,), 0.02)
    res = synth.normal_bf16(rng, (B, N))
    xq = O.q8_1_quantize_bf16(O.rmsnorm(x, nw))
    want = O.gemv_q4k_q8(W, N, K, xq)
    dW, dx, dnw, dxq, dres = dev(W), dev(x), dev(nw), dev(xq), dev(res)
    y = R.DeviceBuffer(B * N * 4)
    ops.gemv_simple(dW.ptr, N, K, dxq.ptr, B, y.ptr)    # few rows: the automatic choice stays on these kernels
    assert_same_bits(y.download(np.float32, (B, N)), want, "Q8_1 blocks in")
    ops.gemv(dxq.ptr, K, B, [ops.gemv_seg(dW.ptr, N, y.ptr, R.BK_EPI_F32)], order=R.BK_GEMV_ORDER_LANES)
    assert_same_bits(y.download(np.float32, (B, N)), want, "Q8_1 blocks in, lane order forced")
    ops.gemv(dxq.ptr, K, B, [ops.gemv_seg(dW.ptr, N, y.ptr, R.BK_EPI_F32)], order=R.BK_GEMV_ORDER_TILE)
    assert_same_bits(y.download(np.float32, (B, N)), O.gemv_q4k_q8_tile(W, N, K, xq) if B >= 16 else want,
                     "Q8_1 blocks in, tile order asked for (the tile kernel from 16 columns on)")
    o = R.DeviceBuffer(B * N * 2)
    ops.gemv(dx.ptr, K, B, [ops.gemv_seg(dW.ptr, N, o.ptr, R.BK_EPI_ADD_BF16, residual=dres.ptr)], prologue=R.BK_PRO_RMSNORM,
             norm_w=dnw.ptr)
    assert_same_bits(o.download(np.uint16, (B, N)), O.epilogue_add(want, res), "bf16 rows in, fused norm, residual out")
    if B % 8 != 1:
        img = R.DeviceBuffer.zeros(ops.staged_bytes(K, B))
        ops.rmsnorm_quant_q8_1(dx.ptr, dnw.ptr, K, B, img.ptr, layout=R.BK_Q8_STAGED)
        ops.gemv(img.ptr, K, B, [ops.gemv_seg(dW.ptr, N, y.ptr, R.BK_EPI_F32)], prologue=R.BK_PRO_STAGED)
        assert_same_bits(y.download(np.float32, (B, N)), want, "grouped staged image in")


@pytest.mark.parametrize("B", [3, 8])
def test_gemv_widest_k_batched(bk, B):
    """K = 17408 (FFN width of the 64-layer configuration) at batch >= 3: too wide for the tensor-core path's
    shared memory, served as column pairs; bf16 prologue, residual epilogue with a column offset."""
    K, N, ld, off = 17408, 200, 256, 40
    rng = np.random.default_rng(70 + B)
    W = synth.q4k_weights(rng, N, K)
    x = synth.normal_bf16(rng, (B, K))
    res = synth.normal_bf16(rng, (B, ld))
    xq = O.q8_1_quantize_bf16(x)
    want = O.epilogue_add(O.gemv_q4k_q8(W, N, K, xq), np.ascontiguousarray(res[:, off:off + N]))
    dW, dx, dres, out = dev(W), dev(x), dev(res), R.DeviceBuffer.zeros(B * ld * 2)
    ops.gemv(dx.ptr, K, B, [ops.gemv_seg(dW.ptr, N, out.ptr, R.BK_EPI_ADD_BF16, ld_out=ld, col_off=off,
                                         residual=dres.ptr)], prologue=R.BK_PRO_BF16)
    got = out.download(np.uint16, (B, ld))
    assert_same_bits(got[:, off:off + N], want, f"gemv K={K} B={B}")
    assert not got[:, :off].any() and not got[:, off + N:].any()
    xq8 = dev(xq)
    y = R.DeviceBuffer(B * N * 4)
    ops.gemv_simple(dW.ptr, N, K, xq8.ptr, B, y.ptr)
    assert_same_bits(y.download(np.float32, (B, N)), O.gemv_q4k_q8(W, N, K, xq), "Q8_1 input, f32 output")


@pytest.mark.parametrize("B", [1, 8])
def test_gemv_fused_prologues_epilogues(bk, B):
    """One launch: RMSNorm prologue, three segments with f32 / bf16 / residual-add epilogues."""
    K, N0, N1, N2 = 2048, 96, 64, 32
    rng = np.random.default_rng(40 + B)
    Ws = [synth.q4k_weights(rng, n, K) for n in (N0, N1, N2)]
    x = synth.normal_bf16(rng, (B, K))
    nw = synth.normal_bf16(rng, (K,), 0.02)
    res = synth.normal_bf16(rng, (B, N2))
    xn = O.rmsnorm(x, nw)
    xq = O.q8_1_quantize_bf16(xn)
    want0 = O.gemv_q4k_q8(Ws[0], N0, K, xq)
    want1 = O.epilogue_cast(O.gemv_q4k_q8(Ws[1], N1, K, xq))
    want2 = O.epilogue_add(O.gemv_q4k_q8(Ws[2], N2, K, xq), res)
    dWs = [dev(w) for w in Ws]
    dx, dnw, dres = dev(x), dev(nw), dev(res)
    o0, o1, o2 = R.DeviceBuffer(B * N0 * 4), R.DeviceBuffer(B * N1 * 2), R.DeviceBuffer(B * N2 * 2)
    ops.gemv(dx.ptr, K, B, [
        ops.gemv_seg(dWs[0].ptr, N0, o0.ptr, R.BK_EPI_F32),
        ops.gemv_seg(dWs[1].ptr, N1, o1.ptr, R.BK_EPI_BF16),
        ops.gemv_seg(dWs[2].ptr, N2, o2.ptr, R.BK_EPI_ADD_BF16, residual=dres.ptr),
    ], prologue=R.BK_PRO_RMSNORM, norm_w=dnw.ptr)
    assert_same_bits(o0.download(np.float32, (B, N0)), want0, "f32 segment")
    assert_same_bits(o1.download(np.uint16, (B, N1)), want1, "bf16 segment")
    assert_same_bits(o2.download(np.uint16, (B, N2)), want2, "add segment")


@pytest.mark.parametrize("B", [1, 4])
def test_gemv_swiglu_bf16_prologue(bk, B):
    K, N = 1024, 200
    rng = np.random.default_rng(50 + B)
    Wg, Wu = synth.q4k_weights(rng, N, K), synth.q4k_weights(rng, N, K)
    x = synth.normal_bf16(rng, (B, K))
    xq = O.q8_1_quantize_bf16(x)
    want = O.swiglu(O.gemv_q4k_q8(Wg, N, K, xq), O.gemv_q4k_q8(Wu, N, K, xq))
    dWg, dWu, dx, out = dev(Wg), dev(Wu), dev(x), R.DeviceBuffer(B * N * 2)
    ops.gemv(dx.ptr, K, B, [ops.gemv_seg(dWg.ptr, N, out.ptr, R.BK_EPI_SWIGLU, W2=dWu.ptr)], prologue=R.BK_PRO_BF16)
    assert_same_bits(out.download(np.uint16, (B, N)), want, "swiglu")


def test_gemv_rejects_bad_arguments(bk):
    with pytest.raises(R.BunkerCudaError) as e:
        ops.gemv_simple(16, 4, 100, 16, 1, 16)  # K not a multiple of 256
    assert e.value.code == R.BK_ERR_ARG
    with pytest.raises(R.BunkerCudaError):
        ops.gemv_simple(16, 4, 256, 16, 65, 16)  # batch beyond 64


def test_gemv_linearity_full_size(bk):
    """Size-independent property at lm_head scale: doubling every Q8_1 scale doubles y exactly."""
    N, K = 151936, 2048
    W, x = synth.gemv_case(N, K, 1, config_id=77)
    xq = O.q8_1_quantize(x)
    xq2 = xq.copy()
    d = xq2[:, :, 32:34].copy().view(np.float16)
    xq2[:, :, 32:34] = (d * np.float16(2)).view(np.uint8)
    dW, a, b = dev(W), dev(xq), dev(xq2)
    ya, yb = R.DeviceBuffer(N * 4), R.DeviceBuffer(N * 4)
    ops.gemv_simple(dW.ptr, N, K, a.ptr, 1, ya.ptr)
    ops.gemv_simple(dW.ptr, N, K, b.ptr, 1, yb.ptr)
    y1, y2 = ya.download(np.float32, (N,)), yb.download(np.float32, (N,))
    assert np.isfinite(y1).all()
    assert_same_bits(y2, y1 * np.float32(2), "linearity")
    rows = np.random.default_rng(0).choice(N, 64, replace=False)
    want = O.gemv_q4k_q8(W[rows], 64, K, xq)
    assert_same_bits(y1[rows].reshape(1, -1), want, "sampled rows")


@pytest.mark.parametrize("B,K,N", [(16, 256, 128), (16, 2048, 131), (17, 2048, 300), (31, 4096, 260), (32, 2048, 1000),
                                   (33, 2048, 150), (64, 6144, 200), (32, 17408, 140),
                                   # row counts that are multiples of 32: weights fed by tiled TMA loads
                                   (16, 1024, 96), (32, 2048, 2080), (24, 768, 4128), (40, 4096, 1056), (32, 6144, 2048)])
def test_gemv_dense_tile_path(bk, B, K, N):
    """16 or more columns of Q8_1 blocks: tcgen05 int8 MMA (one per 32-weight sub-block) with TMEM accumulators.  The
    integer block dots are exact; the f32 chain per (row, column) is the tile order of the oracle, so results are
    bit-identical to it -- for plain f32 output, for several segments with different epilogues in one launch, and
    for the SwiGLU pair."""
    rng = np.random.default_rng(500 + B + K)
    W = synth.q4k_weights(rng, N, K)
    W2 = synth.q4k_weights(rng, N, K)
    x = rng.normal(0, 1, (B, K)).astype(np.float32)
    res = synth.normal_bf16(rng, (B, N))
    xq = O.q8_1_quantize(x)
    want, want2 = O.gemv_q4k_q8_tile(W, N, K, xq), O.gemv_q4k_q8_tile(W2, N, K, xq)
    assert rel_err(want, O.gemv_q4k_q8_plain(W, N, K, xq)) < 1e-3
    dW, dW2, dxq, dres = dev(W), dev(W2), dev(xq), dev(res)
    y = R.DeviceBuffer(B * N * 4)
    T = R.BK_GEMV_ORDER_TILE
    ops.gemv(dxq.ptr, K, B, [ops.gemv_seg(dW.ptr, N, y.ptr, R.BK_EPI_F32)], order=T)
    assert_same_bits(y.download(np.float32, (B, N)), want, "f32 out")
    # three segments in one launch: bf16 cast | residual add | f32, written side by side into rows of 3N
    wide_bf, wide_f = R.DeviceBuffer.zeros(B * 2 * N * 2), R.DeviceBuffer.zeros(B * N * 4)
    segs = [ops.gemv_seg(dW.ptr, N, wide_bf.ptr, R.BK_EPI_BF16, ld_out=2 * N, col_off=0),
            ops.gemv_seg(dW2.ptr, N, wide_bf.ptr, R.BK_EPI_ADD_BF16, ld_out=2 * N, col_off=N, residual=0),
            ops.gemv_seg(dW2.ptr, N, wide_f.ptr, R.BK_EPI_F32)]
    # the residual of segment 1 is indexed like its output: a [B][2N] buffer whose right half holds `res`
    res_wide = np.zeros((B, 2 * N), np.uint16)
    res_wide[:, N:] = res
    dres_w = dev(res_wide)
    segs[1].residual = dres_w.ptr
    ops.gemv(dxq.ptr, K, B, segs, order=T)
    got = wide_bf.download(np.uint16, (B, 2 * N))
    assert_same_bits(got[:, :N], O.epilogue_cast(want), "bf16 segment")
    assert_same_bits(got[:, N:], O.epilogue_add(want2, res), "residual segment")
    assert_same_bits(wide_f.download(np.float32, (B, N)), want2, "f32 segment")
    act = R.DeviceBuffer(B * N * 2)
    ops.gemv(dxq.ptr, K, B, [ops.gemv_seg(dW.ptr, N, act.ptr, R.BK_EPI_SWIGLU, W2=dW2.ptr)], order=T)
    assert_same_bits(act.download(np.uint16, (B, N)), O.swiglu(want, want2), "SwiGLU pair")


def test_gemv_automatic_order_follows_the_row_count(bk):
    """BK_GEMV_ORDER_AUTO at 32 columns: a launch of at least 4096 rows (a SwiGLU pair counts twice), or of at least
    1024 rows with K >= 2048, takes the tile kernel and its order, a smaller one the batch <= 8 kernels and theirs."""
    B, K = 32, 512
    rng = np.random.default_rng(77)
    xq = O.q8_1_quantize(rng.normal(0, 1, (B, K)).astype(np.float32))
    dxq = dev(xq)
    for N, tile in ((4096, True), (4095, False)):
        W = synth.q4k_weights(rng, N, K)
        dW, y = dev(W), R.DeviceBuffer(B * N * 4)
        ops.gemv_simple(dW.ptr, N, K, dxq.ptr, B, y.ptr)
        want = (O.gemv_q4k_q8_tile if tile else O.gemv_q4k_q8)(W, N, K, xq)
        assert_same_bits(y.download(np.float32, (B, N)), want, f"{N} rows")
    K2 = 2048   # from K = 2048 on, 1024 rows are enough (the launch is cut along K over several thread blocks)
    xq2 = O.q8_1_quantize(rng.normal(0, 1, (B, K2)).astype(np.float32))
    dxq2 = dev(xq2)
    for N, tile in ((1024, True), (1023, False)):
        W = synth.q4k_weights(rng, N, K2)
        dW, y = dev(W), R.DeviceBuffer(B * N * 4)
        for _ in range(3):   # the arrival counters of a cut launch reset themselves
            ops.gemv_simple(dW.ptr, N, K2, dxq2.ptr, B, y.ptr)
        want = (O.gemv_q4k_q8_tile if tile else O.gemv_q4k_q8)(W, N, K2, xq2)
        assert_same_bits(y.download(np.float32, (B, N)), want, f"{N} rows, K = 2048")
    N = 2048   # pair: 4096 launch rows
    Wg, Wu = synth.q4k_weights(rng, N, K), synth.q4k_weights(rng, N, K)
    dWg, dWu, act = dev(Wg), dev(Wu), R.DeviceBuffer(B * N * 2)
    ops.gemv(dxq.ptr, K, B, [ops.gemv_seg(dWg.ptr, N, act.ptr, R.BK_EPI_SWIGLU, W2=dWu.ptr)])
    assert_same_bits(act.download(np.uint16, (B, N)),
                     O.swiglu(O.gemv_q4k_q8_tile(Wg, N, K, xq), O.gemv_q4k_q8_tile(Wu, N, K, xq)), "SwiGLU pair of 2 x 2048 rows")
