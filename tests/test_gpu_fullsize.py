"""Parity at the sizes the benchmark runs: the CUDA path against the CPU oracle on row samples of full-size problems.

Y and dX of the linear (and of the gated-MLP block) are independent from token row to token row, so a sample of rows
of a full-size launch can be checked against the oracle evaluated on those rows alone; the adapter gradients reduce
over all tokens and are checked either in full (they only involve rank-r products, cheap on the CPU) or on a smaller
batch.  Tolerance: relative Frobenius error <= 1e-2 (bf16 device path against the fp32 oracle on identical
bf16-rounded inputs), as in the other linear tests.  Seeds and geometries follow BASELINE configs 2, 3 and 5; the
weights are quantised by the package's own quantiser on the device (checked against the oracle's elsewhere) and
dequantised by the oracle on the host.
"""
from __future__ import annotations

import ctypes

import pytest
import torch

from oracle import molt_oracle as oracle
from molt_b200 import _native
from tests.gpu_utils import TOL, assert_clean_status, dense_from_state

pytestmark = pytest.mark.gpu


class FullCase:
    """A weight quantised on the device plus the oracle's dense view of the same bytes."""

    def __init__(self, n, k, rank, *, nested, order="high-first", seed=1337, alpha=None):
        from molt_b200.methods import quantize_nf4

        dev = torch.device("cuda")
        gen = torch.Generator(device=dev).manual_seed(seed)
        w = torch.randn(n, k, device=dev, generator=gen) * 0.02
        self.packed, self.state = quantize_nf4(w, 64, compress_statistics=nested, nibble_order=order)
        del w
        self.n, self.k, self.rank = n, k, rank
        self.scaling = (alpha if alpha is not None else 2.0 * rank) / rank
        self.a = torch.randn(rank, k, device=dev, generator=gen) * 0.01
        self.b = torch.randn(n, rank, device=dev, generator=gen) * 0.01
        self.gen = gen
        self._dense = None

    def dense(self) -> torch.Tensor:
        """deq(W) in fp32 on the host, from the packed bytes and the absmax the device holds."""
        if self._dense is None:
            self._dense = dense_from_state(self.packed, self.state)
        return self._dense

    def desc(self):
        from molt_b200.methods._linear import weight_desc

        return weight_desc(self.packed, self.state)

    def tokens(self, m, width):
        return torch.randn(m, width, device="cuda", generator=self.gen).bfloat16()


@pytest.fixture(scope="module")
def config2(native_library):
    """BASELINE config 2: W [14336, 4096], NF4 blocksize 64, double-quantised absmax, r = 16, alpha = 32."""
    return FullCase(14336, 4096, 16, nested=True)


def _sample_rows(m, count=64, seed=0):
    gen = torch.Generator().manual_seed(seed)
    rows = torch.randperm(m, generator=gen)[:count].sort().values
    # always look at the first and the last row and, where they exist, rows of the last 256-token tile
    extra = torch.tensor([0, m - 1] + ([m - 200, m - 130] if m > 256 else []))
    return torch.unique(torch.cat([rows, extra]))


@pytest.mark.parametrize("m", [64, 256, 1024, 4096, 16384])
def test_config2_forward_rows_against_oracle(config2, m):
    from molt_b200.methods._linear import linear_forward

    c = config2
    x = c.tokens(m, c.k)
    y, _ = linear_forward(c.desc(), x, c.a, c.b, c.scaling, False, _native.PATH_AUTO)
    assert_clean_status()
    rows = _sample_rows(m, seed=m)
    want = oracle.nf4_lora_forward(x[rows.cuda()].float().cpu(), c.dense(), c.a.cpu(), c.b.cpu(), c.scaling)
    assert oracle.rel_frobenius(y[rows.cuda()], want) <= TOL


@pytest.mark.parametrize("m", [1, 16])
def test_config2_gemv_against_oracle(config2, m):
    from molt_b200.methods._linear import linear_forward

    c = config2
    x = c.tokens(m, c.k)
    y, _ = linear_forward(c.desc(), x, c.a, c.b, c.scaling, False, _native.PATH_GEMV)
    assert_clean_status()
    want = oracle.nf4_lora_forward(x.float().cpu(), c.dense(), c.a.cpu(), c.b.cpu(), c.scaling)
    assert oracle.rel_frobenius(y, want) <= TOL


def test_config2_backward_at_4096_tokens_on_every_schedule(config2):
    """The benchmarked backward, as the library schedules it by itself (tall tiles on this device), and on the other
    schedules the same call can take: short tiles with the last wave split along the contraction (256 tiles on 74 CTA
    pairs) and short tiles on the plain schedule.  dX on sampled rows against the oracle, dA and dB in full."""
    from molt_b200.methods._linear import linear_backward

    c, m = config2, 4096
    x, dy = c.tokens(m, c.k), c.tokens(m, c.n)
    dx, da, db = linear_backward(c.desc(), x, dy, c.a, c.b, c.scaling, None, True, True, path=_native.PATH_AUTO)
    short = _native.PATH_TCGEN05 | _native.PATH_SHORT_TILES
    dx_split, _, _ = linear_backward(c.desc(), x, dy, c.a, c.b, c.scaling, None, True, False, path=short)
    dx_plain, _, _ = linear_backward(c.desc(), x, dy, c.a, c.b, c.scaling, None, True, False,
                                     path=short | _native.PATH_NO_SPLIT)
    assert_clean_status()
    assert not torch.equal(dx_split, dx_plain), "short tiles were expected to split their last wave at this size"
    assert oracle.rel_frobenius(dx_split, dx_plain.float()) < 1e-3
    assert oracle.rel_frobenius(dx, dx_plain.float()) < 1e-3
    rows = _sample_rows(m, count=64, seed=7)
    # the last wave's tiles are the last in band order: rows of the last band, last column tiles; sample there too
    rows = torch.unique(torch.cat([rows, torch.arange(m - 2048, m, 97)]))
    a, b = c.a.cpu(), c.b.cpu()
    dy_rows = dy[rows.cuda()].float().cpu()
    want_dx = dy_rows @ c.dense() + c.scaling * ((dy_rows @ b) @ a)
    assert oracle.rel_frobenius(dx[rows.cuda()], want_dx) <= TOL
    assert oracle.rel_frobenius(dx_split[rows.cuda()], want_dx) <= TOL
    xf, dyf = x.float().cpu(), dy.float().cpu()
    want_da = c.scaling * (dyf @ b).t() @ xf          # reference streaming/engine.py:41-44
    want_db = c.scaling * dyf.t() @ (xf @ a.t())
    assert oracle.rel_frobenius(da, want_da) <= TOL and oracle.rel_frobenius(db, want_db) <= TOL


@pytest.mark.parametrize("n,k", [(4096, 4096), (14336, 4096), (4096, 14336)])
def test_config5_rank64_nested(native_library, n, k):
    """BASELINE config 5's projections: rank 64, alpha 128, double-quantised absmax; forward and backward in full at
    256 tokens."""
    from molt_b200.methods._linear import linear_backward, linear_forward

    c, m = FullCase(n, k, 64, nested=True, alpha=128.0, seed=n + k), 256
    x, dy = c.tokens(m, k), c.tokens(m, n)
    y, t = linear_forward(c.desc(), x, c.a, c.b, c.scaling, True, _native.PATH_AUTO)
    dx, da, db = linear_backward(c.desc(), x, dy, c.a, c.b, c.scaling, t, True, True, path=_native.PATH_AUTO)
    assert_clean_status()
    w, a, b = c.dense(), c.a.cpu(), c.b.cpu()
    want_y = oracle.nf4_lora_forward(x.float().cpu(), w, a, b, c.scaling)
    want_dx, want_da, want_db = oracle.nf4_lora_backward(x.float().cpu(), dy.float().cpu(), w, a, b, c.scaling)
    for got, want in ((y, want_y), (dx, want_dx), (da, want_da), (db, want_db)):
        assert oracle.rel_frobenius(got, want) <= TOL


def _config3_block(seed=1337):
    from molt_b200.modules import GatedMLP, NF4LoRALinear

    hidden, inter, rank = 1536, 8960, 16
    cases = [FullCase(inter, hidden, rank, nested=False, order="low-first", seed=seed),
             FullCase(inter, hidden, rank, nested=False, order="low-first", seed=seed + 1),
             FullCase(hidden, inter, rank, nested=False, order="low-first", seed=seed + 2)]
    projs = []
    for c in cases:
        lin = NF4LoRALinear(c.packed, c.state, rank, 32.0)
        with torch.no_grad():
            lin.lora_A["default"].weight.copy_(c.a)
            lin.lora_B["default"].weight.copy_(c.b)
        projs.append(lin)
    dense = [oracle.OracleProjection(c.dense(), c.a.cpu(), c.b.cpu(), 2.0) for c in cases]
    return GatedMLP(*projs), dense, cases[0].gen


def test_config3_block_at_full_size(native_library):
    """BASELINE config 3: gate, up [8960, 1536], down [1536, 8960], r = 16, 8192 tokens, `up` replayed in backward.
    y and dx on sampled rows of the 8192-token launch; all six adapter gradients on a 256-token batch."""
    mlp, dense, gen = _config3_block()
    m, hidden = 8192, 1536
    x = torch.randn(m, hidden, device="cuda", generator=gen).bfloat16()
    dy = torch.randn(m, hidden, device="cuda", generator=gen).bfloat16()
    xin = x.detach().requires_grad_()
    y = mlp.fused(xin, rematerialize_up=True)
    y.backward(dy)
    assert_clean_status()
    rows = _sample_rows(m, count=48, seed=3).cuda()
    ref = oracle.gated_mlp_fwd_bwd(x[rows].float().cpu(), dy[rows].float().cpu(), *dense)
    assert oracle.rel_frobenius(y[rows], ref["y"]) <= TOL
    assert oracle.rel_frobenius(xin.grad[rows], ref["dx"]) <= TOL
    # adapter gradients: a 256-token batch, replayed and kept `up`
    for p in mlp.parameters():
        p.grad = None
    xs, dys = x[:256].detach().requires_grad_(), dy[:256]
    mlp.fused(xs, rematerialize_up=True).backward(dys)
    assert_clean_status()
    ref = oracle.gated_mlp_fwd_bwd(xs.detach().float().cpu(), dys.float().cpu(), *dense)
    for name in ("gate", "up", "down"):
        proj = getattr(mlp, f"{name}_proj")
        assert oracle.rel_frobenius(proj.lora_A["default"].weight.grad, ref[f"{name}_a"]) <= TOL, name
        assert oracle.rel_frobenius(proj.lora_B["default"].weight.grad, ref[f"{name}_b"]) <= TOL, name


def test_fused_lora_input_gradient_on_the_tensor_cores(native_library):
    """packed_nf4_lora_backward_input at a config-3 shape (down projection, 512 tokens, r = 16) runs the tcgen05 kernel
    with the low-rank term as one more contraction block; against the oracle's statement of
    reference methods/nf4_backward.py:127-136."""
    from molt_b200.methods import packed_nf4_lora_backward_input

    c, m = FullCase(1536, 8960, 16, nested=False, seed=5), 512
    dy = c.tokens(m, c.n)
    lora_grad = torch.randn(m, c.rank, device="cuda", generator=c.gen).bfloat16()
    launches = _native.library().molt_launch_count()
    for a in (c.a, c.a.bfloat16()):     # fp32 master and bf16 compute copy
        got = packed_nf4_lora_backward_input(dy, c.packed, c.state, lora_grad, a, 0.125)
        want = oracle.packed_backward_input(dy.float().cpu(), c.dense(), lora_grad.float().cpu(),
                                            a.bfloat16().float().cpu(), 0.125)
        assert oracle.rel_frobenius(got, want) <= TOL
    assert_clean_status()
    # two calls, each: operand prep + tcgen05 GEMM (+ at most the fix-up of a split last wave)
    assert _native.library().molt_launch_count() - launches <= 6
    lib = _native.library()
    ws = _native.workspace(lib.molt_workspace_bytes(_native.OP_DX, m, c.n, c.k, c.rank), dy.device)
    out = torch.empty(m, c.k, device="cuda", dtype=torch.bfloat16)
    desc = c.desc()
    _native.check(lib.molt_nf4_dx(ctypes.byref(desc), dy.data_ptr(), lora_grad.data_ptr(), c.a.data_ptr(),
                                  _native.DTYPE_F32, 0.125, c.rank, out.data_ptr(), m, ws.data_ptr(), ws.numel(),
                                  _native.PATH_TCGEN05, _native.stream_handle()))
    assert torch.equal(out, got) or oracle.rel_frobenius(out, got.float()) < 2e-3   # fp32 master vs its bf16 copy
