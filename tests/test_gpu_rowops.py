"""GPU parity tests of the row kernels (LayerNorm, softmax family, embedding sum) against the CPU oracle,
with the edge cases the reference tests (ragged sizes, fully masked rows, -inf entries) and size-independent
properties at the sizes of the row-op sweep."""
import numpy as np
import pytest

from conftest import relerr
from sptorch_b200.backend import BF16, F32, bf16_bits_to_f32, f32_to_bf16_bits

pytestmark = pytest.mark.gpu


def _bf16(x):
    return bf16_bits_to_f32(f32_to_bf16_bits(x)).reshape(np.shape(x))


@pytest.mark.parametrize("rows,dim", [(1, 1), (5, 3), (64, 128), (9, 768), (300, 768), (5, 2048), (3, 4096), (2, 5000), (2, 8192), (1, 10001)])
def test_layernorm_f32_vs_oracle(backend, oracle, rows, dim):
    rng = np.random.default_rng(rows * 7 + dim)
    x = (rng.standard_normal((rows, dim)) * 3 + 0.5).astype(np.float32)
    g = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    b = (0.1 * rng.standard_normal(dim)).astype(np.float32)
    # tree reduction vs the reference's sequential sums: f32 rounding only
    assert relerr(backend.layernorm(x, g, b), oracle.layernorm(x, g, b)) <= 2e-6


@pytest.mark.parametrize("rows,dim", [(64, 128), (9, 768), (5, 2048), (3, 4096), (2, 5000)])
def test_layernorm_bf16_vs_oracle(backend, oracle, rows, dim):
    rng = np.random.default_rng(dim)
    x = _bf16((rng.standard_normal((rows, dim)) * 3 + 0.5).astype(np.float32))
    g = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    b = (0.1 * rng.standard_normal(dim)).astype(np.float32)
    ref = oracle.layernorm(x, g, b)
    out = backend.layernorm(x, g, b, dtype=BF16)
    assert np.abs(out - ref).max() <= 2 ** -8 * np.abs(ref).max()      # one bf16 rounding of the output


@pytest.mark.parametrize("rows,dim", [(1, 768), (17, 1024), (4096, 768), (4099, 768), (4111, 1024), (4100, 2048), (65536, 768)])
def test_layernorm_bf16_pipelined_kernel_vs_oracle(backend, oracle, rows, dim):
    """bf16 rows of 768 / 1024 / 2048 run the kernel that streams blocks of rows through shared memory with bulk asynchronous
    copies; row counts that are not a multiple of the 16 (8) rows of a block exercise the ragged last block.  Every output
    element against the oracle within one bf16 rounding."""
    rng = np.random.default_rng(rows + dim)
    x = _bf16((rng.standard_normal((rows, dim)) * 3 + 0.5).astype(np.float32))
    g = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    b = (0.1 * rng.standard_normal(dim)).astype(np.float32)
    ref = oracle.layernorm(x, g, b)
    out = backend.layernorm(x, g, b, dtype=BF16)
    assert out.shape == ref.shape
    assert np.abs(out - ref).max() <= 2 ** -8 * np.abs(ref).max()
    # rows are independent: the same rows inside a different row count (another block phase, another CTA) give the same bits
    if rows > 3:
        sub = backend.layernorm(x[5:4101 + 5] if rows > 5000 else x[3:], g, b, dtype=BF16)
        assert np.array_equal(sub, out[5:4101 + 5] if rows > 5000 else out[3:])


def test_layernorm_mean_zero_property_full_size(backend):
    # crates/nn/src/lib.rs:3239-3262 at the row-op sweep's size (65536 x 768): gamma=1, beta=0 -> row mean ~ 0, var ~ 1
    rows, dim = 65536, 768
    x = (np.random.default_rng(0).standard_normal((rows, dim)) * 3 + 0.5).astype(np.float32)
    y = backend.layernorm(x, np.ones(dim, np.float32), np.zeros(dim, np.float32))
    assert np.abs(y.mean(-1)).max() < 1e-5
    assert np.abs(y.var(-1) - 1).max() < 1e-3


@pytest.mark.parametrize("rows,cols", [(1, 1), (5, 3), (64, 64), (33, 1000), (7, 768), (3, 4096), (2, 8192), (2, 10000), (3, 7)])
def test_softmax_vs_oracle(backend, oracle, rows, cols):
    s = (np.random.default_rng(cols).standard_normal((rows, cols)) * 2).astype(np.float32)
    out = backend.softmax_f32(s, rows, cols)
    assert relerr(out, oracle.softmax(s)) <= 4e-6       # tree sum vs sequential sum of up to 10^4 terms, 2-ulp expf
    assert np.abs(out.sum(-1) - 1).max() < 1e-5


def test_softmax_with_minus_inf_entries(backend, oracle):
    s = np.random.default_rng(1).standard_normal((4, 64)).astype(np.float32)
    s[:, 10:] = -np.inf
    out = backend.softmax_f32(s, 4, 64)
    assert (out[:, 10:] == 0).all() and relerr(out, oracle.softmax(s)) <= 2e-6


@pytest.mark.parametrize("bh,t", [(3, 8), (2, 64), (2, 100), (1, 1024), (2, 37), (1, 1), (2, 12), (1, 2048)])
def test_causal_softmax_vs_oracle(backend, oracle, bh, t):
    s = (np.random.default_rng(t).standard_normal((bh, t, t)) * 2).astype(np.float32)
    out = backend.causal_softmax(s, 0.125)
    ref = oracle.causal_softmax(s, 0.125)
    assert relerr(out, ref) <= 2e-6
    assert (np.triu(out, 1) == 0).all()                       # masked entries are exact zeros
    assert np.array_equal(out[:, 0, 0], np.ones(bh, np.float32))   # row 0 is one-hot (crates/nn/src/lib.rs:612-632)


def test_causal_softmax_bf16(backend, oracle):
    s = _bf16((np.random.default_rng(3).standard_normal((2, 128, 128)) * 2).astype(np.float32))
    out = backend.causal_softmax(s, 0.125, dtype=BF16)
    ref = oracle.causal_softmax(s, 0.125)
    assert np.abs(out - ref).max() <= 2 ** -8
    assert (np.triu(out, 1) == 0).all()


@pytest.mark.parametrize("bh,t", [(8, 256), (5, 512), (3, 1024), (2, 2048), (1, 256)])
def test_causal_softmax_bf16_pipelined_kernel(backend, oracle, bh, t):
    """bf16 matrices of 256 / 512 / 1024 / 2048 columns with at least 2048 rows run the kernel that streams row prefixes through a
    ring of shared-memory stages (the last case, 256 rows, stays on the register kernel): against the oracle on the same
    bf16-rounded scores, exact zeros above the diagonal, rows summing to one within the output rounding, a block of rows that
    ends a matrix followed by one that begins the next."""
    s = _bf16((np.random.default_rng(bh + t).standard_normal((bh, t, t)) * 2).astype(np.float32))
    out = backend.causal_softmax(s, 0.125, dtype=BF16)
    ref = oracle.causal_softmax(s, 0.125)
    assert np.abs(out - ref).max() <= 2 ** -8
    assert (np.triu(out, 1) == 0).all()
    assert np.array_equal(out[:, 0, 0], np.ones(bh, np.float32))
    assert np.abs(out.sum(-1) - 1).max() <= 2e-2


def test_causal_softmax_rows_sum_to_one_full_size(backend):
    # the row-op sweep's shape per (batch, head): T = 1024; here 24 matrices (100 MB)
    s = (np.random.default_rng(4).standard_normal((24, 1024, 1024)) * 2).astype(np.float32)
    out = backend.causal_softmax(s, 1.0)
    assert np.abs(out.sum(-1) - 1).max() < 1e-5 and (np.triu(out, 1) == 0).all()


def test_masked_softmax_vs_oracle(backend, oracle):
    rng = np.random.default_rng(5)
    a = rng.standard_normal((6, 50)).astype(np.float32)
    keep = rng.random((6, 50)) < 0.6
    keep[2] = False                                           # a row with nothing kept stays all zero
    out = backend.masked_softmax(a, keep)
    assert relerr(out, oracle.masked_softmax(a, keep)) <= 2e-6
    assert (out[2] == 0).all() and (out[~keep] == 0).all()
    # KAT: crates/core-ops/src/lib.rs:2561-2574
    d = backend.masked_softmax(np.array([[1, 2], [3, 4]], np.float32), [True, False, True, True]).ravel()
    assert d[0] == 1.0 and d[1] == 0.0 and abs(d[2] + d[3] - 1) < 1e-6
    # rank-1 rule: everything kept is -inf -> uniform over kept
    r1 = backend.masked_softmax(np.array([-np.inf, -np.inf, 1.0], np.float32), [True, True, False])
    assert r1.tolist() == [0.5, 0.5, 0.0]


def test_embedding_sum_vs_oracle(backend, oracle):
    rng = np.random.default_rng(6)
    tok = rng.standard_normal((40, 32)).astype(np.float32); pos = rng.standard_normal((16, 32)).astype(np.float32)
    ids = rng.integers(0, 40, 48)
    ref = oracle.binary("add", oracle.embedding(tok, ids), oracle.embedding(pos, np.arange(48) % 16))
    assert np.array_equal(backend.embedding_sum(tok, pos, ids, 16).ravel(), ref.ravel())
    out = backend.embedding_sum(_bf16(tok), _bf16(pos), ids, 16, dtype=BF16)
    refb = _bf16(tok)[ids] + _bf16(pos)[np.arange(48) % 16]
    assert np.abs(out - refb).max() <= 2 ** -8 * np.abs(refb).max()      # one bf16 rounding of the sum


def test_gelu_bf16_and_f32(backend, oracle):
    x = np.random.default_rng(7).standard_normal(70001).astype(np.float32)
    assert np.abs(backend.gelu(x) - oracle.unary("gelu", x)).max() <= 1e-6
    xb = _bf16(x)
    assert np.abs(backend.gelu(xb, dtype=BF16) - oracle.unary("gelu", xb)).max() <= 2 ** -8 * 4
