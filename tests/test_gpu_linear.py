"""NF4 + LoRA linear forward/backward through the C ABI on every kernel path, against the CPU oracle."""
from __future__ import annotations

import pytest
import torch

from oracle import molt_oracle as oracle
from molt_b200 import _native
from tests.conftest import load_golden
from tests.gpu_utils import TOL, assert_clean_status, make_case, oracle_results, run_backward, run_forward

pytestmark = pytest.mark.gpu

PATHS = {"general": _native.PATH_GENERAL, "tcgen05": _native.PATH_TCGEN05}


def _check_all(case, path):
    y_ref, dx_ref, da_ref, db_ref = oracle_results(case)
    y, t = run_forward(case, path, keep_t=True)
    dx, da, db = run_backward(case, path, t)
    torch.cuda.synchronize()
    assert_clean_status()
    errors = {"y": oracle.rel_frobenius(y, y_ref), "dx": oracle.rel_frobenius(dx, dx_ref),
              "da": oracle.rel_frobenius(da, da_ref), "db": oracle.rel_frobenius(db, db_ref)}
    assert all(v <= TOL for v in errors.values()), errors
    # backward without the saved low-rank product recomputes it
    dx2, da2, db2 = run_backward(case, path, None)
    assert torch.equal(dx2, dx) and torch.equal(da2, da) and torch.equal(db2, db)
    return errors


@pytest.mark.parametrize("name", ["lin_8x8_r2", "lin_96x64_r8", "lin_70x65_r7", "lin_256x128_r16"])
def test_general_path_matches_reference_fixture(native_library, name):
    """Inputs AND expected outputs come from the reference's own eager path (tests/golden)."""
    from molt_b200.methods._linear import linear_backward, linear_forward, weight_desc
    from molt_b200.methods.quant_state import QuantState

    fx = load_golden(name)
    n, k = fx["w"].shape
    state = QuantState(absmax=torch.from_numpy(fx["scales"]).cuda(), shape=(n, k), blocksize=int(fx["block"]),
                       nibble_order="low-first")
    packed = torch.from_numpy(fx["packed"]).cuda()
    desc = weight_desc(packed, state)
    x = torch.from_numpy(fx["x"]).cuda().bfloat16()
    dy = torch.from_numpy(fx["dy"]).cuda().bfloat16()
    a, b = torch.from_numpy(fx["a"]).cuda(), torch.from_numpy(fx["b"]).cuda()
    s = float(fx["scaling"])
    path = _native.PATH_AUTO if (n % 64 == 0 and k % 64 == 0) else _native.PATH_GENERAL
    y, t = linear_forward(desc, x, a, b, s, True, path)
    dx, da, db = linear_backward(desc, x, dy, a, b, s, t, True, True, path=path)
    assert_clean_status()
    for got, key in ((y, "y"), (dx, "dx"), (da, "da"), (db, "db")):
        assert oracle.rel_frobenius(got, torch.from_numpy(fx[key])) <= TOL, key


@pytest.mark.parametrize("path", ["general", "tcgen05"])
@pytest.mark.parametrize("n,k", [(96, 64), (256, 1536), (1536, 1536)])
@pytest.mark.parametrize("scaling", [0.125, 2.0])
def test_reference_geometries(native_library, path, n, k, scaling):
    # geometries, M=256, r=8 and seed 941 of reference tests/kernels/test_nf4_lora.py:14-45 (width, out_width swapped
    # into [out, in]); 64 -> 96 is the (64, 96) case
    case = make_case(n, k, 256, 8, seed=941, scaling=scaling, order="high-first", nested=True, w_std=1.0, ab_std=0.05)
    if path == "tcgen05" and (n % 64 or k % 64):
        pytest.skip("unaligned geometry: covered by the general kernels")
    _check_all(case, PATHS[path])


@pytest.mark.parametrize("n,k", [(8960, 1536), (1536, 8960)])
def test_reference_mlp_geometries_tcgen05(native_library, n, k):
    case = make_case(n, k, 256, 8, seed=941, scaling=0.3, order="high-first", nested=True)
    _check_all(case, PATHS["tcgen05"])


def test_config1_single_linear(native_library):
    """BASELINE config 1: W [4864, 896], r=16, alpha=32, X [512, 896]; MOLT's own format (low-first, fp32 absmax)."""
    case = make_case(4864, 896, 512, 16, seed=1337)
    errors = _check_all(case, _native.PATH_AUTO)
    assert max(errors.values()) < 5e-3


@pytest.mark.parametrize("m", [1, 5, 127, 129, 300])
def test_ragged_token_counts(native_library, m):
    case = make_case(256, 192, m, 16, seed=7 + m)
    _check_all(case, PATHS["tcgen05"])


@pytest.mark.parametrize("rank", [1, 7, 16, 33, 64])
def test_rank_tails_on_both_paths(native_library, rank):
    case = make_case(320, 128, 96, rank, seed=943, scaling=0.125, ab_std=0.1)
    _check_all(case, PATHS["tcgen05"])
    _check_all(case, PATHS["general"])


def test_dimension_tails_use_the_general_kernels(native_library):
    # W [70, 65], dY [5, 70], rank 7, seeds of reference tests/kernels/test_nf4_lora.py:106-143
    case = make_case(70, 65, 5, 7, seed=942, scaling=0.125, order="high-first", w_std=1.0)
    _check_all(case, _native.PATH_AUTO)
    with pytest.raises(Exception, match="tcgen05"):
        run_forward(case, _native.PATH_TCGEN05)


@pytest.mark.parametrize("n,k,m", [(64, 64, 256), (64, 128, 300), (128, 64, 40), (192, 64, 513)])
def test_short_contractions(native_library, n, k, m):
    """One or two contraction blocks per tile: shorter than the pipeline's lead of codes over activations."""
    case = make_case(n, k, m, 8, seed=n + k + m)
    _check_all(case, PATHS["tcgen05"])


@pytest.mark.parametrize("n,k", [(2560, 1024), (1024, 2560)])
def test_split_last_wave(native_library, n, k):
    """80 output tiles (of the short kind) on 74 CTA pairs (forward for the first shape, backward for the second): the six tiles of the
    last wave are cut along the contraction, leave the GEMM as fp32 partial tiles and are summed by the fix-up kernel
    (forced here: for tiles this short the library would keep the plain schedule).  Results must match the oracle
    and, up to the order of fp32 additions, the plain schedule."""
    case = make_case(n, k, 2048, 16, seed=n + k, nested=True, order="high-first")
    short = PATHS["tcgen05"] | _native.PATH_SHORT_TILES
    split, plain = short | _native.PATH_FORCE_SPLIT, short | _native.PATH_NO_SPLIT
    _check_all(case, split)
    y_split, _ = run_forward(case, split)
    dx_split, da_split, db_split = run_backward(case, split)
    y_plain, _ = run_forward(case, plain)
    dx_plain, da_plain, db_plain = run_backward(case, plain)
    assert oracle.rel_frobenius(y_split, y_plain.float()) < 1e-3
    assert oracle.rel_frobenius(dx_split, dx_plain.float()) < 1e-3
    assert not (torch.equal(y_split, y_plain) and torch.equal(dx_split, dx_plain))   # the split schedule really ran
    assert torch.equal(da_split, da_plain) and torch.equal(db_split, db_plain)
    assert_clean_status()


@pytest.mark.parametrize("height", ["tall", "short"])
@pytest.mark.parametrize("n,k,m,rank", [(512, 320, 300, 16), (256, 128, 513, 8), (1536, 256, 1100, 64), (320, 1536, 2048, 16)])
def test_tile_heights(native_library, height, n, k, m, rank):
    """Both tile heights of the tensor-core GEMM (512 and 256 tokens per CTA pair), forced, on token counts that leave
    the last tile ragged in either; results must match the oracle and each other up to fp32 summation order."""
    flag = _native.PATH_TALL_TILES if height == "tall" else _native.PATH_SHORT_TILES
    case = make_case(n, k, m, rank, seed=n + m, nested=(k % 256 == 0), order="high-first")
    _check_all(case, PATHS["tcgen05"] | flag)
    y_this, _ = run_forward(case, PATHS["tcgen05"] | flag)
    y_auto, _ = run_forward(case, PATHS["tcgen05"])
    assert oracle.rel_frobenius(y_this, y_auto.float()) < 1e-3


@pytest.mark.parametrize("n,k", [(2560, 1024), (1024, 2560)])
def test_split_last_wave_of_tall_tiles(native_library, n, k):
    """80 tall tiles (4096 tokens) on 74 CTA pairs: the six tiles of the last wave are cut along the contraction; both
    accumulators of every part go out as fp32 partial tiles and the fix-up kernel adds them."""
    case = make_case(n, k, 4096, 16, seed=n + k + 1, nested=True, order="high-first")
    split = PATHS["tcgen05"] | _native.PATH_FORCE_SPLIT | _native.PATH_TALL_TILES
    plain = PATHS["tcgen05"] | _native.PATH_NO_SPLIT | _native.PATH_TALL_TILES
    _check_all(case, split)
    y_split, _ = run_forward(case, split)
    dx_split, da_split, db_split = run_backward(case, split)
    y_plain, _ = run_forward(case, plain)
    dx_plain, da_plain, db_plain = run_backward(case, plain)
    assert oracle.rel_frobenius(y_split, y_plain.float()) < 1e-3
    assert oracle.rel_frobenius(dx_split, dx_plain.float()) < 1e-3
    assert not (torch.equal(y_split, y_plain) and torch.equal(dx_split, dx_plain))   # the split schedule really ran
    assert_clean_status()


def test_empty_batch(native_library):
    case = make_case(128, 64, 0, 8)
    y, _ = run_forward(case)
    assert y.shape == (0, 128)
    dx, da, db = run_backward(case)
    assert dx.shape == (0, 64) and torch.count_nonzero(da) == 0 and torch.count_nonzero(db) == 0


def test_tcgen05_forward_equals_general_forward_closely(native_library):
    case = make_case(512, 256, 384, 16, seed=5)
    y_fast, _ = run_forward(case, PATHS["tcgen05"])
    y_slow, _ = run_forward(case, PATHS["general"])
    assert oracle.rel_frobenius(y_fast, y_slow.float()) < 4e-3


def test_forward_linearity_at_full_size(native_library):
    """Size-independent property at BASELINE config 2's weight (14336 x 4096, nested absmax), M = 4096:
    rows are independent, so the forward of a row subset equals the subset of the forward -- bit for bit on the plain
    tile schedule, and up to the order of two fp32 additions where the tiles of the last wave are split."""
    case = make_case(14336, 4096, 64, 16, seed=1337, nested=True, order="high-first")
    gen = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(4096, 4096, device="cuda", generator=gen).bfloat16()
    from molt_b200.methods._linear import linear_forward, weight_desc

    desc = weight_desc(case.packed, case.state)
    a, b = case.a.cuda(), case.b.cuda()
    full, _ = linear_forward(desc, x, a, b, 2.0, False, _native.PATH_TCGEN05)
    part, _ = linear_forward(desc, x[1024:1536].contiguous(), a, b, 2.0, False, _native.PATH_TCGEN05)
    assert_clean_status()
    differing = (full[1024:1536] != part).float().mean().item()
    assert differing < 0.02 and oracle.rel_frobenius(full[1024:1536], part.float()) < 1e-3
    plain = _native.PATH_TCGEN05 | _native.PATH_NO_SPLIT
    full_plain, _ = linear_forward(desc, x, a, b, 2.0, False, plain)
    part_plain, _ = linear_forward(desc, x[1024:1536].contiguous(), a, b, 2.0, False, plain)
    assert_clean_status()
    assert torch.equal(full_plain[1024:1536], part_plain)
    # and a 64-row slice against the oracle
    y_ref = oracle.nf4_lora_forward(x[:64].float().cpu(), case.weight, case.a, case.b, 2.0)
    assert oracle.rel_frobenius(full[:64], y_ref) <= TOL


@pytest.mark.parametrize("m", [1, 3, 8, 16])
@pytest.mark.parametrize("n,k,nested", [(256, 128, False), (1536, 896, False), (4864, 896, False), (512, 4096, True),
                                        (256, 8960, True)])
def test_gemv_path(native_library, m, n, k, nested):
    case = make_case(n, k, m, 16, seed=11 + m, nested=nested, order="high-first" if nested else "low-first")
    y, _ = run_forward(case, _native.PATH_GEMV)
    y_ref = oracle.nf4_lora_forward(case.x, case.weight, case.a, case.b, case.scaling)
    assert oracle.rel_frobenius(y, y_ref) <= TOL
    y_again, _ = run_forward(case, _native.PATH_GEMV)
    assert torch.equal(y, y_again)  # deterministic, tickets left clean


def test_gemv_wide_and_ragged_rows(native_library):
    """Rows wider than one pass of the streaming kernel's K-slices (K = 16384: 256 absmax blocks) and a block count that
    no slice layout divides evenly (K = 16448: 257 blocks); both must match the oracle."""
    case = make_case(128, 16384, 4, 16, seed=77, nested=True, order="high-first")
    y, _ = run_forward(case, _native.PATH_GEMV)
    y_ref = oracle.nf4_lora_forward(case.x, case.weight, case.a, case.b, case.scaling)
    assert oracle.rel_frobenius(y, y_ref) <= TOL
    wide = make_case(128, 16448, 11, 16, seed=78)
    y_wide, _ = run_forward(wide, _native.PATH_GEMV)
    y_wide_ref = oracle.nf4_lora_forward(wide.x, wide.weight, wide.a, wide.b, wide.scaling)
    assert oracle.rel_frobenius(y_wide, y_wide_ref) <= TOL
    assert oracle.rel_frobenius(run_forward(wide, _native.PATH_AUTO)[0], y_wide_ref) <= TOL   # 11 tokens: the few-token kernel
    assert_clean_status()


@pytest.mark.parametrize("n,k,m,rank", [(64, 64, 1, 1), (192, 1536, 9, 64), (8960, 1536, 16, 16), (1536, 8960, 5, 16),
                                        (24 * 8 * 148, 128, 7, 8)])
def test_gemv_plans(native_library, n, k, m, rank):
    """Shapes that exercise the streaming kernel's plans: a single row group per CTA, rank 64, 24 and 140 absmax blocks
    per row (slices of 2 and 3 blocks, several passes), more row groups than one wave of CTAs holds, and t_out."""
    case = make_case(n, k, m, rank, seed=n + k + m, nested=(k % 256 == 0), order="high-first")
    y, t = run_forward(case, _native.PATH_GEMV, keep_t=True)
    y_ref = oracle.nf4_lora_forward(case.x, case.weight, case.a, case.b, case.scaling)
    assert oracle.rel_frobenius(y, y_ref) <= TOL
    t_ref = case.x @ case.a.bfloat16().float().t()
    assert oracle.rel_frobenius(t[:, :rank], t_ref) <= TOL and torch.count_nonzero(t[:, rank:]) == 0
    assert_clean_status()


def test_gemv_is_the_auto_path_for_few_tokens(native_library):
    case = make_case(512, 256, 4, 8, seed=21)
    y_auto, _ = run_forward(case, _native.PATH_AUTO)
    y_gemv, _ = run_forward(case, _native.PATH_GEMV)
    assert torch.equal(y_auto, y_gemv)
    with pytest.raises(Exception, match="16 tokens"):
        run_forward(make_case(512, 256, 17, 8), _native.PATH_GEMV)
    # 9 to 128 tokens: the few-token kernel; above: the GEMM
    for tokens in (9, 40, 128):
        case = make_case(512, 256, tokens, 8, seed=22)
        assert torch.equal(run_forward(case, _native.PATH_AUTO)[0], run_forward(case, _native.PATH_FEW_TOKENS)[0])
    case = make_case(512, 256, 129, 8, seed=23)
    assert torch.equal(run_forward(case, _native.PATH_AUTO)[0], run_forward(case, _native.PATH_TCGEN05)[0])
    with pytest.raises(Exception, match="128 tokens"):
        run_forward(case, _native.PATH_FEW_TOKENS)


def test_packed_backward_input_operators(native_library):
    from molt_b200.methods import packed_nf4_backward_input, packed_nf4_lora_backward_input

    for (n, k, m, r, seed) in [(70, 65, 5, 7, 943), (256, 192, 40, 16, 9)]:
        case = make_case(n, k, m, r, seed=seed, order="high-first", w_std=1.0, scaling=0.125)
        dy = case.dy.cuda().bfloat16()
        base = packed_nf4_backward_input(dy, case.packed, case.state)
        want = oracle.packed_backward_input(case.dy, case.weight)
        assert oracle.rel_frobenius(base, want) <= TOL
        gen = torch.Generator().manual_seed(seed)
        lora_grad = torch.randn(m, r, generator=gen).bfloat16()
        fused = packed_nf4_lora_backward_input(dy, case.packed, case.state, lora_grad.cuda(), case.a.cuda(), 0.125)
        want = oracle.packed_backward_input(case.dy, case.weight, lora_grad.float(), case.a.bfloat16().float(), 0.125)
        assert oracle.rel_frobenius(fused, want) <= TOL
    with pytest.raises(ValueError, match="width"):
        packed_nf4_backward_input(torch.zeros(2, 3, device="cuda", dtype=torch.bfloat16), case.packed, case.state)


@pytest.mark.parametrize("exact", [False, True])
@pytest.mark.parametrize("m", [1, 5, 16, 17, 33, 64, 100, 128])
@pytest.mark.parametrize("n,k,rank,nested,order", [(1536, 1024, 16, True, "high-first"), (320, 192, 7, False, "low-first"),
                                                   (2048, 4096, 64, True, "low-first")])
def test_few_token_path(native_library, m, n, k, rank, nested, order, exact):
    """Forward with at most 128 tokens on the swapped-operand tcgen05 kernel (weight rows are the MMA rows): parts of a
    row tile computed by different CTAs, a last tile with 64 valid rows, ranks that are not multiples of 16, both absmax
    forms (the nested one resolved inside the kernel), and both decodes: the table decode (bf16 codebook pair times
    bf16 absmax) and the one with the dequantiser's bits.
    Must match the oracle, and the low-rank product it returns must match the one of the tensor-core path."""
    case = make_case(n, k, m, rank, seed=n + k + m, nested=nested, order=order)
    path = _native.PATH_FEW_TOKENS | (_native.PATH_EXACT_DECODE if exact else 0)
    y_ref = oracle_results(case)[0]
    y, t = run_forward(case, path, keep_t=True)
    torch.cuda.synchronize()
    assert_clean_status()
    assert oracle.rel_frobenius(y, y_ref) <= TOL
    y2, t2 = run_forward(case, _native.PATH_TCGEN05, keep_t=True)
    assert oracle.rel_frobenius(y, y2.float()) <= (2e-3 if exact else 6e-3)
    assert oracle.rel_frobenius(t[:, :rank].float(), t2[:, :rank].float()) <= 4e-3
    assert not t[:, rank:].any()
    # deterministic: a second call gives the same bits
    y3, _ = run_forward(case, path, keep_t=False)
    assert torch.equal(y3, y)


@pytest.mark.parametrize("n,k,m,rank,nested", [(1536, 1024, 300, 16, False), (320, 192, 40, 7, True),
                                               (2560, 1024, 2048, 64, False), (1536, 8960, 5, 16, False)])
def test_lora_shadows_give_the_same_bits_as_the_per_call_conversion(native_library, n, k, m, rank, nested):
    """The bf16 adapter operands kept by the optimizer's side (reference methods/lora_shadow.py:19-141) stand in for the
    conversion in front of each call: same kernels, same operands, so the results are identical, on every path."""
    from molt_b200.methods._linear import LoraShadows, ShadowTable, linear_backward, linear_forward, weight_desc_for_tokens

    case = make_case(n, k, m, rank, nested=nested, seed=77)
    desc = weight_desc_for_tokens(case.packed, case.state, m)
    a, b = case.a.cuda(), case.b.cuda()
    x, dy = case.x.cuda().bfloat16(), case.dy.cuda().bfloat16()
    other = LoraShadows(torch.randn(5, 64, device="cuda"), torch.randn(128, 5, device="cuda"), 0.5)
    shadow = LoraShadows(a, b, case.scaling)
    ShadowTable([other, shadow]).refresh()       # two adapters of different shapes in one launch
    rp = (rank + 15) // 16 * 16
    assert torch.equal(shadow.a16[:rank], a.bfloat16()) and not shadow.a16[rank:].any()
    assert torch.equal(shadow.bs[:, :rank], (case.scaling * b).bfloat16()) and not shadow.bs[:, rank:].any()
    assert torch.equal(shadow.bt[:rank], (case.scaling * b).bfloat16().t()) and shadow.bt.shape == (rp, n)
    assert torch.equal(other.a16[:5], other.lora_a.bfloat16())
    for path in (_native.PATH_AUTO, _native.PATH_TCGEN05):
        y0, t0 = linear_forward(desc, x, a, b, case.scaling, True, path)
        y1, t1 = linear_forward(desc, x, a, b, case.scaling, True, path, shadow=shadow)
        assert torch.equal(y0, y1) and torch.equal(t0, t1)
        g0 = linear_backward(desc, x, dy, a, b, case.scaling, t0, True, True, path=path)
        g1 = linear_backward(desc, x, dy, a, b, case.scaling, t1, True, True, path=path, shadow=shadow)
        assert all(torch.equal(u, v) for u, v in zip(g0, g1))
    assert_clean_status()
    y_ref = oracle_results(case)[0]
    assert oracle.rel_frobenius(y1, y_ref) <= TOL
    if not nested:   # one launch fewer per call on the tensor-core path: the operand preparation is gone
        count = native_library.molt_launch_count
        c0 = count()
        linear_forward(desc, x, a, b, case.scaling, True, _native.PATH_TCGEN05)
        c1 = count()
        linear_forward(desc, x, a, b, case.scaling, True, _native.PATH_TCGEN05, shadow=shadow)
        c2 = count()
        linear_backward(desc, x, dy, a, b, case.scaling, t0, True, True, path=_native.PATH_TCGEN05)
        c3 = count()
        linear_backward(desc, x, dy, a, b, case.scaling, t0, True, True, path=_native.PATH_TCGEN05, shadow=shadow)
        c4 = count()
        assert (c2 - c1, c4 - c3) == (c1 - c0 - 1, c3 - c2 - 1)
    # stale shadows are what the kernels use: the owner has to refresh after changing the masters
    a.mul_(2.0)
    y_stale, _ = linear_forward(desc, x, a, b, case.scaling, False, _native.PATH_TCGEN05, shadow=shadow)
    assert torch.equal(y_stale, y1)
    ShadowTable([shadow]).refresh()
    y_new, _ = linear_forward(desc, x, a, b, case.scaling, False, _native.PATH_TCGEN05, shadow=shadow)
    y_plain, _ = linear_forward(desc, x, a, b, case.scaling, False, _native.PATH_TCGEN05)
    assert torch.equal(y_new, y_plain) and not torch.equal(y_new, y1)


@pytest.mark.parametrize("n,k,m,rank", [(1536, 1024, 300, 16), (2560, 1024, 2048, 8), (256, 4096, 700, 64)])
def test_gemm_reads_a_double_quantised_absmax_itself(native_library, n, k, m, rank):
    """The tensor-core GEMM's decoders resolve code2[u8] * absmax2 + offset on the fly (no fp32 copy of the absmax is
    made first): same bits as the resolved array, so forward and backward equal the calls on the resolved descriptor."""
    from molt_b200.methods._linear import linear_backward, linear_forward, weight_desc
    from molt_b200.methods.quant_state import QuantState

    case = make_case(n, k, m, rank, nested=True, order="high-first", seed=99)
    nested_desc = weight_desc(case.packed, case.state)
    plain = QuantState(absmax=case.scales_f32.cuda(), shape=(n, k), nibble_order="high-first")
    plain_desc = weight_desc(case.packed, plain)
    a, b = case.a.cuda(), case.b.cuda()
    x, dy = case.x.cuda().bfloat16(), case.dy.cuda().bfloat16()
    count = native_library.molt_launch_count
    results = []
    for desc in (nested_desc, plain_desc):
        c0 = count()
        y, t = linear_forward(desc, x, a, b, case.scaling, True, _native.PATH_TCGEN05)
        grads = linear_backward(desc, x, dy, a, b, case.scaling, t, True, True, path=_native.PATH_TCGEN05)
        results.append((y, *grads, count() - c0))
    assert all(torch.equal(u, v) for u, v in zip(results[0][:4], results[1][:4]))
    assert results[0][4] == results[1][4]          # and no extra launch for the nested form
    assert_clean_status()
    y_ref, dx_ref, _, _ = oracle_results(case)
    assert oracle.rel_frobenius(results[0][0], y_ref) <= TOL and oracle.rel_frobenius(results[0][1], dx_ref) <= TOL


def _fuzz_cases(count, seed):
    gen = torch.Generator().manual_seed(seed)

    def pick(values):
        return values[int(torch.randint(0, len(values), (1,), generator=gen))]

    cases = []
    for index in range(count):
        n = 64 * pick([1, 2, 3, 5, 8, 13, 24, 40])
        k = 64 * pick([1, 2, 3, 4, 7, 16, 24, 36])
        m = pick([1, 2, 7, 8, 9, 16, 31, 64, 100, 128, 129, 255, 257, 511, 640, 1100])
        rank = pick([1, 4, 8, 16, 17, 32, 48, 64])
        cases.append((n, k, m, rank, bool(pick([0, 1])), pick(["low-first", "high-first"]), pick([0.25, 1.0, 2.0]), 5000 + index))
    return cases


@pytest.mark.parametrize("n,k,m,rank,nested,order,scaling,seed", _fuzz_cases(36, 20261125))
def test_seeded_random_shapes_on_the_auto_path(native_library, n, k, m, rank, nested, order, scaling, seed):
    """Randomly drawn (seeded) aligned shapes, token counts on both sides of every path boundary, ranks with tails, both
    nibble orders and both absmax forms, on whatever path AUTO takes: Y, dX, dA, dB against the oracle."""
    case = make_case(n, k, m, rank, seed=seed, scaling=scaling, nested=nested, order=order)
    y_ref, dx_ref, da_ref, db_ref = oracle_results(case)
    y, t = run_forward(case, _native.PATH_AUTO, keep_t=True)
    dx, da, db = run_backward(case, _native.PATH_AUTO, t)
    torch.cuda.synchronize()
    assert_clean_status()
    errors = {"y": oracle.rel_frobenius(y, y_ref), "dx": oracle.rel_frobenius(dx, dx_ref),
              "da": oracle.rel_frobenius(da, da_ref), "db": oracle.rel_frobenius(db, db_ref)}
    assert all(v <= TOL for v in errors.values()), errors
