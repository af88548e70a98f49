"""The CPU oracle against vectors produced by the reference's own code
(tests/golden/make_golden.py).  Integer/byte outputs must match bit for bit."""
import numpy as np
import pytest

from oracle import wush_oracle as wo


def test_rtn_e2m1_sweep(golden):
    vals, codes = wo.rtn_e2m1(golden["e2m1_in"])
    assert np.array_equal(vals, golden["e2m1_vals"])
    assert np.array_equal(np.signbit(vals), np.signbit(golden["e2m1_vals"]))
    assert np.array_equal(wo.pack_e2m1(codes), golden["e2m1_packed"])
    assert np.array_equal(wo.unpack_e2m1(golden["e2m1_packed"]), golden["e2m1_unpacked"])


def test_scale_casts(golden):
    assert np.array_equal(wo.cast_e8m0(golden["cast_in"]), golden["cast_e8m0"])
    assert np.array_equal(wo.cast_e4m3(golden["cast_e4m3_in"]), golden["cast_e4m3"])


@pytest.mark.parametrize("fmt", ["mxfp4", "nvfp4"])
@pytest.mark.parametrize("case", ["edge", "rand_f32", "rand_bf16"])
def test_rtn_xxfp4(golden, fmt, case):
    x = golden[f"{fmt}_{case}_in"]
    r = wo.rtn_xxfp4(x, fmt)
    assert np.array_equal(r["scale_quant"], golden[f"{fmt}_{case}_scale_quant"])
    assert np.array_equal(r["e2m1"], golden[f"{fmt}_{case}_e2m1"])
    want = golden[f"{fmt}_{case}_fake_quant"]
    got = r["fake_quant"]
    if case == "rand_bf16":
        got = wo.round_to_bf16(got)          # the reference casts back to x.dtype
    elif case != "edge" or True:
        got = got.astype(np.float32).astype(np.float64) if case != "rand_bf16" else got
    assert np.array_equal(np.nan_to_num(got, nan=-777.0), np.nan_to_num(want, nan=-777.0))
    deq = wo.dequant_xxfp4(golden[f"{fmt}_{case}_e2m1"], golden[f"{fmt}_{case}_scale_quant"], fmt)
    assert np.array_equal(np.nan_to_num(deq, nan=-777.0), np.nan_to_num(golden[f"{fmt}_{case}_dequant"], nan=-777.0))


@pytest.mark.parametrize("grp", [32, 16])
def test_transforms(golden, grp):
    basis, y, t_ref = golden[f"tf{grp}_basis"], golden[f"tf{grp}_y"], golden[f"tf{grp}_wush"]
    assert np.array_equal(wo.get_transform(basis[:grp, :grp], y[:grp], "hadamard"), golden[f"tf{grp}_hadamard"])
    for i in range(t_ref.shape[0]):
        sl = slice(i * grp, (i + 1) * grp)
        t = wo.get_transform(basis[sl, sl], y[sl], "wush")
        # the transform is rounded to bf16 (8 significant bits): the two LAPACK paths agree to
        # ~1e-13 before rounding, so after rounding all but a handful of entries are identical
        assert np.mean(t != t_ref[i]) < 5e-3
        assert np.allclose(t, t_ref[i], rtol=2 ** -7, atol=1e-6)
        # sign-convention-free property: (T B^T)(T B^T)^T = Had diag(s) Had^T
        tb, tb_ref = t @ basis[sl, sl].T, t_ref[i] @ basis[sl, sl].T
        gram, gram_ref = tb @ tb.T, tb_ref @ tb_ref.T
        assert np.abs(gram - gram_ref).max() <= 2e-2 * np.abs(gram_ref).max()
    x = golden[f"tf{grp}_x"]
    bt = wo.block_transform(x, t_ref)
    assert np.array_equal(bt.astype(np.float32).astype(np.float64), golden[f"tf{grp}_bt_f32"])
    assert np.array_equal(wo.round_to_bf16(bt), golden[f"tf{grp}_bt_bf16"])
    fmt = "mxfp4" if grp == 32 else "nvfp4"
    r = wo.fused_transform_quant(x, wo.transform_to_matrix(t_ref), fmt)
    assert np.array_equal(r["e2m1"], golden[f"tf{grp}_q_e2m1"])
    assert np.array_equal(r["scale_quant"], golden[f"tf{grp}_q_scale_quant"])


def test_hessian_running_mean(golden):
    xs = list(golden["hess_in"])
    h = wo.wush_update_sequence(xs)
    ref = golden["hess_out_f32"].astype(np.float64)
    assert np.abs(h - ref).max() <= 1e-5 * np.abs(ref).max()
    flat = np.concatenate([x.reshape(-1, x.shape[-1]) for x in xs])
    assert np.allclose(h, wo.hessian_xtx(flat) / flat.shape[0], rtol=1e-12, atol=1e-12)


def test_roundtrips():
    rng = np.random.default_rng(0)
    codes = rng.integers(0, 16, size=(7, 64), dtype=np.uint8)
    assert np.array_equal(wo.unpack_e2m1_codes(wo.pack_e2m1(codes)), codes)
    t = rng.standard_normal((4, 32, 32))
    assert np.array_equal(wo.matrix_to_transform(wo.transform_to_matrix(t)), t)
    # unpacking the packed codes and scales reproduces the fake-quantized tensor
    x = rng.standard_normal((16, 128))
    for fmt in ("mxfp4", "nvfp4"):
        q1 = wo.rtn_xxfp4(x, fmt)
        assert np.array_equal(wo.dequant_xxfp4(q1["e2m1"], q1["scale_quant"], fmt), q1["fake_quant"])
        # frozen scales reproduce the same codes (the GPTQ column steps rely on this)
        q2 = wo.rtn_xxfp4(x, fmt, existing_scale=q1["scale_quant"])
        assert np.array_equal(q1["e2m1"], q2["e2m1"])


def test_to_blocked_layout():
    rows, cols = 200, 10
    s = (np.arange(rows)[:, None] * 16 + np.arange(cols)[None, :]).astype(np.uint16)
    blk = wo.to_blocked(s)
    assert blk.size == 256 * 12
    for r, c in [(0, 0), (31, 3), (32, 0), (127, 3), (128, 4), (199, 9), (130, 5)]:
        tile = (r // 128) * 3 + c // 4
        off = tile * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + c % 4
        assert blk[off] == s[r, c]


# ---- "quest" scaling: the reference's Triton kernel run on CPU by the Triton interpreter -------------------------

def _quest_golden():
    import os
    return np.load(os.path.join(os.path.dirname(__file__), "golden", "quest_vectors.npz"))


@pytest.mark.parametrize("transform", ["identity", "hadamard", "hadamard64", "hadamard128"])
def test_quest_matches_triton_kernel(transform):
    d = _quest_golden()
    x = d["x"]
    mat = np.eye(32, dtype=np.float32) if transform == "identity" else d[transform]
    y = (x.reshape(-1, mat.shape[0]) @ mat).reshape(x.shape)  # float32, as the interpreter's tl.dot
    r = wo.quest_mxfp4(y)
    want = d[f"{transform}_quest_out"]
    assert np.array_equal(r["fake_quant"], want)
    assert np.array_equal(np.signbit(r["fake_quant"]), np.signbit(want))
    assert np.array_equal(r["clip_mask"], d[f"{transform}_quest_clip"])
    assert 0.90 < r["clip_mask"].mean() < 0.98                # the outlier channel and the scaled rows do clip
    # codes and scale bytes rebuild the same values
    vals = wo.E2M1_VALUES[wo.unpack_e2m1_codes(r["e2m1"])].reshape(-1, 32)
    scale = np.exp2(r["scale_quant"].astype(np.float64) - 127).reshape(-1, 1)
    assert np.array_equal((vals * scale).reshape(x.shape), want.astype(np.float64))


@pytest.mark.parametrize("transform", ["identity", "hadamard", "hadamard64", "hadamard128"])
def test_absmax_agrees_with_triton_kernel_off_ties(transform):
    """The abs-max branch of the same Triton kernel against the restatement of the torch quantizer: identical
    except where a scaled value sits exactly on a rounding boundary (Triton rounds those toward zero, the torch
    quantizer to the even code); an all-zero group comes out as -0 with its clip flags cleared (0/0 there)."""
    d = _quest_golden()
    x = d["x"].astype(np.float64)
    mat = np.eye(32) if transform == "identity" else d[transform].astype(np.float64)
    if mat.shape[0] == 32:
        r = wo.fused_transform_quant(x, mat, "mxfp4")
    else:                                      # wide transform, then the quantizer on float32-rounded values
        y = wo.wide_transform(x, mat).astype(np.float32).astype(np.float64)
        r = wo.rtn_xxfp4(y, "mxfp4")
        r["transformed"] = y
    want = d[f"{transform}_absmax_out"].astype(np.float64)
    got = r["fake_quant"]
    scale = np.exp2(r["scale_quant"].astype(np.float64) - 127)
    scaled = np.abs(r["transformed"].reshape(-1, 32) * 3.0 / scale.reshape(-1, 1)).reshape(x.shape)
    tie = np.isin(scaled, [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
    ok = np.isclose(got, want, rtol=1e-6, atol=0.0) | tie          # 4/3 * 2^e is rounded to float32 there
    assert ok.all() and not np.isnan(want).any()
    clip = d[f"{transform}_absmax_clip"]
    if mat.shape[0] == 32:                     # wider transforms mix the all-zero group with its neighbours
        assert not clip[8, :32].any() and clip.sum() == clip.size - 32
    else:
        assert clip.all()
