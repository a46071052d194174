"""GPU parity tests of the tcgen05 GEMM behind nn::Linear and attention, against the CPU oracle."""
import numpy as np
import pytest

from conftest import elementwise_excess, parity_record, relerr
from sptorch_b200.backend import BF16, EPI_GELU, F32, MM_BF16, MM_F32, MM_TF32, bf16_bits_to_f32, f32_to_bf16_bits

pytestmark = pytest.mark.gpu


def _bf16(x):
    return bf16_bits_to_f32(f32_to_bf16_bits(x)).reshape(np.shape(x))


SHAPES = [(1, 8, 8), (128, 64, 64), (128, 64, 256), (129, 72, 257), (256, 768, 768), (512, 768, 3072), (300, 136, 200),
          (512, 3072, 768), (64, 4096, 512), (1000, 40, 50257 // 64)]


@pytest.mark.parametrize("M,K,N", SHAPES)
def test_linear_tf32_and_bf16_vs_oracle(backend, oracle, M, K, N):
    rng = np.random.default_rng(M + K + N)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (0.02 * rng.standard_normal((N, K))).astype(np.float32)
    b = (0.01 * rng.standard_normal(N)).astype(np.float32)
    ref = oracle.linear(x, w, b, fast=2)
    assert relerr(backend.linear(x, w, b, mode=MM_TF32), ref) <= 2e-3          # north star: TF32 within 2e-3
    assert relerr(backend.linear(x, w, b, mode=MM_BF16), ref) <= 2e-2          # north star: bf16 within 2e-2
    assert relerr(backend.linear(x, w, b, mode=MM_F32), ref) <= 5e-6           # CUDA-core f32 FMA
    # bf16 path against the oracle fed the same bf16-rounded operands: only the output rounding remains
    refb = oracle.linear(_bf16(x), _bf16(w), b, fast=2)
    assert relerr(backend.linear(x, w, b, mode=MM_BF16), refb) <= 2 ** -8 * 1.1
    assert relerr(backend.linear(x, w, b, mode=MM_BF16, out_dtype=F32), refb) <= 1e-5


@pytest.mark.parametrize("M", [4096, 16384])
@pytest.mark.parametrize("K,N", [(768, 768), (768, 3072), (3072, 768), (4096, 4096)])
def test_linear_sweep_shapes_vs_oracle(backend, oracle, M, K, N):
    """The standalone Linear sweep at its large row counts with the inputs it specifies (x ~ N(0,1), W ~ N(0,0.02), b ~ N(0,0.01),
    seeded per shape): every output element of the bf16 and the TF32 path against the oracle's f32 product (blocked, all host
    threads; no rows are left out)."""
    from sptorch_b200 import synth
    seed = 1000 * (M // 512) + K + N
    x = synth.normal(seed, M * K).reshape(M, K)
    w = synth.normal(seed + 1, N * K, std=0.02).reshape(N, K)
    b = synth.normal(seed + 2, N, std=0.01)
    ref = oracle.linear(x, w, b, fast=1)
    for mode, tol, name in ((MM_TF32, 2e-3, "tf32"), (MM_BF16, 2e-2, "bf16")):
        out = backend.linear(x, w, b, mode=mode)
        err = relerr(out, ref)
        outside, worst = elementwise_excess(out, ref, tol)
        parity_record(f"linear {M}x{K}->{N} {name}", relerr=err, elementwise_worst=worst)
        assert err <= tol, (name, err)
        assert worst <= 1.0, (name, outside, worst)


def test_linear_fused_epilogues(backend, oracle):
    rng = np.random.default_rng(1)
    M, K, N = 200, 128, 328
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (0.05 * rng.standard_normal((N, K))).astype(np.float32)
    b = (0.1 * rng.standard_normal(N)).astype(np.float32)
    r = rng.standard_normal((M, N)).astype(np.float32)
    lin = oracle.linear(x, w, b, fast=2)
    ref = oracle.unary("gelu", lin) + r
    assert relerr(backend.linear(x, w, b, residual=r, epilogue=EPI_GELU, mode=MM_TF32), ref) <= 2e-3
    assert relerr(backend.linear(x, w, b, residual=r, epilogue=EPI_GELU, mode=MM_F32), ref) <= 5e-6
    assert relerr(backend.linear(x, w, b, residual=r, epilogue=EPI_GELU, mode=MM_BF16), ref) <= 2e-2
    assert relerr(backend.linear(x, w, None, alpha=0.5, mode=MM_TF32), 0.5 * oracle.linear(x, w, None, fast=2)) <= 2e-3


@pytest.mark.parametrize("M", [1, 3, 8, 16, 17, 33, 64])
@pytest.mark.parametrize("K,N", [(768, 768), (768, 2304), (3072, 768), (256, 50257 // 8), (96, 40)])
def test_linear_with_few_rows_vs_oracle(backend, oracle, M, K, N):
    """At most 64 input rows in bf16 (the projections of a decode step) run the weight-streaming kernel instead of 128-row
    tiles: against the oracle on the same bf16-rounded operands (only the output rounding remains), with the fused epilogues,
    and exactly on one-hot rows, where out[m, n] must be W[n, k_m]: every k position of an activation row has to meet the same
    k position of every weight row, ragged row and column counts included."""
    rng = np.random.default_rng(1000 * M + K + N)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (0.02 * rng.standard_normal((N, K))).astype(np.float32)
    b = (0.01 * rng.standard_normal(N)).astype(np.float32)
    r = rng.standard_normal((M, N)).astype(np.float32)
    refb = oracle.linear(_bf16(x), _bf16(w), b, fast=2)
    assert relerr(backend.linear(x, w, b, mode=MM_BF16), refb) <= 2 ** -8 * 1.1
    assert relerr(backend.linear(x, w, b, mode=MM_BF16), oracle.linear(x, w, b, fast=2)) <= 2e-2
    ref = oracle.unary("gelu", refb) + _bf16(r)
    assert relerr(backend.linear(x, w, b, residual=r, epilogue=EPI_GELU, mode=MM_BF16), ref) <= 2 ** -8 * 1.1
    assert relerr(backend.linear(x, w, None, alpha=0.5, mode=MM_BF16), 0.5 * oracle.linear(_bf16(x), _bf16(w), None, fast=2)) <= 2 ** -8 * 1.1
    ks = rng.integers(0, K, M)
    onehot = np.zeros((M, K), np.float32)
    onehot[np.arange(M), ks] = 1.0
    wi = rng.integers(-64, 65, (N, K)).astype(np.float32)
    assert np.array_equal(backend.linear(onehot, wi, mode=MM_BF16), wi[:, ks].T)


def test_linear_with_few_rows_on_tcgen05_tiles():
    """Row counts up to 64 take the weight-streaming kernel by default; SPTORCH_B200_FEW_ROWS=0 (read once per process, hence the
    child process) sends them through the 128-row tcgen05 tiles instead, which must agree with the oracle too."""
    import os, subprocess, sys, textwrap
    code = textwrap.dedent("""
        import numpy as np
        from sptorch_b200.backend import FfiBackend, MM_BF16, EPI_GELU, bf16_bits_to_f32, f32_to_bf16_bits
        from oracle import binding as oracle
        b = FfiBackend.load()
        r16 = lambda x: bf16_bits_to_f32(f32_to_bf16_bits(x)).reshape(np.shape(x))
        rel = lambda a, r: float(np.linalg.norm(a - r) / np.linalg.norm(r))
        for M, K, N in [(33, 768, 768), (64, 768, 2304), (64, 3072, 768), (48, 256, 6282)]:
            rng = np.random.default_rng(M + K + N)
            x = rng.standard_normal((M, K)).astype(np.float32)
            w = (0.02 * rng.standard_normal((N, K))).astype(np.float32)
            bias = (0.01 * rng.standard_normal(N)).astype(np.float32)
            res = rng.standard_normal((M, N)).astype(np.float32)
            ref = oracle.linear(r16(x), r16(w), bias, fast=2)
            assert rel(b.linear(x, w, bias, mode=MM_BF16), ref) <= 2 ** -8 * 1.1
            assert rel(b.linear(x, w, bias, residual=res, epilogue=EPI_GELU, mode=MM_BF16), oracle.unary("gelu", ref) + r16(res)) <= 2 ** -8 * 1.1
            ks = rng.integers(0, K, M)
            onehot = np.zeros((M, K), np.float32)
            onehot[np.arange(M), ks] = 1.0
            wi = rng.integers(-64, 65, (N, K)).astype(np.float32)
            assert np.array_equal(b.linear(onehot, wi, mode=MM_BF16), wi[:, ks].T)
        b.close()
        print("ok")
    """)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, SPTORCH_B200_FEW_ROWS="0", PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
    out = subprocess.run([sys.executable, "-c", code], cwd=root, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and "ok" in out.stdout, out.stdout + out.stderr


def test_linear_is_linear_at_full_size(backend):
    """Size-independent property at a shape of the standalone Linear sweep (M 4096, K 768, N 3072): f(x1 + x2) = f(x1) + f(x2) and
    integer-valued operands give exact integers."""
    rng = np.random.default_rng(2)
    M, K, N = 4096, 768, 3072
    x = rng.integers(-4, 5, (M, K)).astype(np.float32)
    w = rng.integers(-2, 3, (N, K)).astype(np.float32)
    out = backend.linear(x, w, mode=MM_BF16, out_dtype=F32)
    ref = (x.astype(np.int32) @ w.astype(np.int32).T).astype(np.float32)
    assert np.array_equal(out, ref)                       # exact: every product and partial sum is a small integer
    assert np.array_equal(backend.linear(x, w, mode=MM_TF32), ref)


@pytest.mark.parametrize("M,K,N", [(1100, 512, 50304), (8320, 512, 50304), (300, 64, 1000), (4100, 64, 328)])
def test_tile_rasterisation_covers_every_tile_exactly_once(backend, M, K, N):
    """Integer-valued operands make every output exact, so a tile that is skipped, doubled or misplaced by the tile decode shows
    up as a wrong integer.  Shapes: a B operand above 48 MB (64-tile bands: one ragged band, then a full band plus a ragged
    one) and small operands (8-tile bands with ragged tails)."""
    rng = np.random.default_rng(M + N)
    x = rng.integers(-4, 5, (M, K)).astype(np.float32)
    w = rng.integers(-2, 3, (N, K)).astype(np.float32)
    ref = x @ w.T                                            # exact in f32: |sum| <= 8 * 512
    assert np.array_equal(backend.linear(x, w, mode=MM_BF16, out_dtype=F32), ref)
    assert np.array_equal(backend.linear(x, w, mode=MM_TF32), ref)


@pytest.mark.parametrize("M,K,N", [(129, 64, 129), (256, 64, 256), (640, 200, 328), (1000, 768, 1000), (2048, 3072, 768), (4100, 136, 50257 // 16)])
def test_pair_tiles_equal_single_cta_tiles(backend, oracle, M, K, N):
    """Wide problems run on CTA pairs (256 x 256 tiles, one MMA over two SMs).  Every output element is still the same
    k-ordered f32 accumulation, so the result must be bit-identical to the one-CTA kernel's; both are checked against the
    oracle.  Shapes cover a second row half that is partly or wholly outside the matrix and ragged N."""
    rng = np.random.default_rng(M * 7 + N)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (0.05 * rng.standard_normal((N, K))).astype(np.float32)
    b = (0.1 * rng.standard_normal(N)).astype(np.float32)
    r = rng.standard_normal((M, N)).astype(np.float32)
    ref = oracle.unary("gelu", oracle.linear(x, w, b, fast=2)) + r
    try:
        outs = {}
        for pair in (1, 0, 3):
            backend._check(backend.lib.sptorch_ext_set_gemm_pair(pair), "set_gemm_pair")
            outs[pair] = [backend.linear(x, w, b, residual=r, epilogue=EPI_GELU, mode=MM_TF32),
                          backend.linear(x, w, b, residual=r, epilogue=EPI_GELU, mode=MM_BF16),
                          backend.linear(x, w, b, mode=MM_BF16, out_dtype=F32)]
    finally:
        backend.lib.sptorch_ext_set_gemm_pair(3)           # the default: pairs where they measured faster
    for a, c, d in zip(outs[1], outs[0], outs[3]):
        assert np.array_equal(a, c) and np.array_equal(d, c)
    assert relerr(outs[1][0], ref) <= 2e-3
    assert relerr(outs[1][1], ref) <= 2e-2


@pytest.mark.parametrize("B,T,H,hd", [(2, 64, 4, 32), (1, 256, 2, 64), (2, 128, 2, 128), (1, 1024, 1, 64), (3, 8, 2, 32)])
def test_attention_vs_oracle(backend, oracle, B, T, H, hd):
    rng = np.random.default_rng(B * T + hd)
    d = H * hd
    q, k, v = (rng.standard_normal((B, T, d)).astype(np.float32) for _ in range(3))
    eye = np.eye(d, dtype=np.float32)
    # oracle: the reference's MHA with identity projections is exactly the attention core
    ref = np.stack([_mha_core(oracle, q[i], k[i], v[i], H) for i in range(B)])
    assert relerr(backend.attention_causal(q, k, v, H, dtype=F32), ref) <= 2e-3
    assert relerr(backend.attention_causal(q, k, v, H, dtype=BF16), ref) <= 2e-2
    del eye


def _mha_core(oracle, q, k, v, H):
    T, d = q.shape
    hd = d // H
    out = np.empty_like(q)
    for h in range(H):
        sl = slice(h * hd, (h + 1) * hd)
        s = oracle.matmul(q[:, sl], oracle.transpose(k[:, sl]), f64=True)[None]
        p = oracle.causal_softmax(s, 1.0 / np.sqrt(np.float32(hd)))[0]
        out[:, sl] = oracle.matmul(p, v[:, sl], f64=True)
    return out


@pytest.mark.parametrize("B,T,H,hd", [(1, 8, 1, 64), (2, 128, 3, 64), (1, 200, 2, 64), (2, 384, 2, 64), (1, 1024, 2, 64), (1, 136, 2, 128), (2, 512, 1, 128)])
def test_fused_attention_matches_materialised_and_oracle(backend, oracle, B, T, H, hd):
    """The fused kernel (scores never leave the SM) against the three-launch materialised form and the oracle,
    including sequence lengths that are not a multiple of the 128-row tile."""
    rng = np.random.default_rng(T + hd)
    d = H * hd
    q, k, v = (_bf16(rng.standard_normal((B, T, d)).astype(np.float32)) for _ in range(3))
    fused = backend.attention_causal(q, k, v, H, dtype=BF16)
    backend.lib.sptorch_ext_set_attention_mode(1)
    try:
        mat = backend.attention_causal(q, k, v, H, dtype=BF16)
    finally:
        backend.lib.sptorch_ext_set_attention_mode(0)
    ref = np.stack([_mha_core(oracle, q[i], k[i], v[i], H) for i in range(B)])
    assert relerr(fused, ref) <= 2e-2 and relerr(mat, ref) <= 2e-2
    assert relerr(fused, ref) <= 1.5 * 2 ** -8           # one bf16 rounding of P and of the output
    assert np.array_equal(fused[:, 0, :], v[:, 0, :])    # row 0 attends only to itself: output = V[0] exactly


@pytest.mark.parametrize("T,hd", [(256, 64), (384, 128), (200, 64)])
def test_fused_attention_with_steeply_rising_scores(backend, oracle, T, hd):
    """Scores that grow by far more than 2^8 from one 32-key chunk to the next (key j = 8 (j // 4) u, query = u): the running row maximum
    of the fused kernel moves at every chunk, so everything accumulated under the old maximum -- the row sum, the output in TMEM and
    the part of P already written for the current tile -- is rescaled each time.  The softmax is then concentrated on the last
    few visible keys; the result must still match the oracle within one bf16 rounding of P and of the output."""
    rng = np.random.default_rng(T + hd)
    H = 2
    u = np.where(rng.random(hd) < 0.5, -0.125, 0.125).astype(np.float32)
    q = np.tile(u, (1, T, H)).astype(np.float32)
    k = np.concatenate([(8.0 * (j // 4)) * np.tile(u, H)[None, :] for j in range(T)])[None].astype(np.float32)
    v = _bf16(rng.standard_normal((1, T, H * hd)).astype(np.float32))
    assert np.array_equal(_bf16(k), k)                     # the keys are exact in bf16
    fused = backend.attention_causal(q, k, v, H, dtype=BF16)
    ref = _mha_core(oracle, q[0], k[0], v[0], H)[None]
    assert relerr(fused, ref) <= 1.5 * 2 ** -8
    # and the other way round: falling scores never move the maximum after the first chunk
    k2 = k[:, ::-1].copy()
    fused2 = backend.attention_causal(q, k2, v, H, dtype=BF16)
    ref2 = _mha_core(oracle, q[0], k2[0], v[0], H)[None]
    assert relerr(fused2, ref2) <= 1.5 * 2 ** -8
