"""Generate tests/golden/*.npz by RUNNING THE REFERENCE'S OWN CODE on CPU.

Usage (needs the reference checkout; writes next to this file):

    python tests/golden/make_golden.py /path/to/WUSH          # reference_vectors.npz
    python tests/golden/make_golden.py /path/to/WUSH sweep    # sweep_vectors.npz (column sweep)
    TRITON_INTERPRET=1 python tests/golden/make_golden.py /path/to/WUSH quest   # quest_vectors.npz

The reference has no numeric tests or fixtures of its own, so these files -- outputs of
its pure-torch quantizer (src/quantization/wush_gptq.py) on small seeded inputs and
hand-picked edge cases -- are what pins the CPU oracle in ``oracle/wush_oracle.py``.
Nothing here is imported at test time; the tests only read the .npz files.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _import_reference(root: str):
    sys.dont_write_bytecode = True
    os.chdir(root)                     # the reference imports `inference_lib...` from cwd
    sys.path.insert(0, root)
    from src.quantization import wush_gptq  # noqa: WPS433
    return wush_gptq


def _u8(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.uint8).numpy().copy()


def _quant(ref, x: torch.Tensor, fmt: str) -> dict:
    kw = dict(mxfp4=dict(group_size=32, scale_dtype=torch.float8_e8m0fnu, scale_scale=4., global_scale=3.),
              nvfp4=dict(group_size=16, scale_dtype=torch.float8_e4m3fn, scale_scale=6., global_scale=10.))[fmt]
    r = ref.rtn_xxfp4(x, fp4_rounding_mode="even", **kw)
    deq = ref.dequant_xxfp4(r["e2m1"], r["scale_quant"], r["global_scale"], dtype=torch.float64)
    return dict(fake_quant=r["fake_quant"].to(torch.float64).numpy(), e2m1=_u8(r["e2m1"]),
                scale_quant=_u8(r["scale_quant"]), dequant=deq.numpy())


def edge_inputs(group: int) -> torch.Tensor:
    """Rows of one or two groups that exercise ties, zeros, signs, tiny and huge
    magnitudes.  float32 so every value is exact."""
    rows = []
    base = torch.zeros(group)
    rows.append(base.clone())                                      # all-zero group
    r = base.clone(); r[0] = 1.0; rows.append(r)                   # single non-zero
    r = base.clone(); r[0] = -1.0; r[1] = -0.0; rows.append(r)
    # every E2M1 rounding boundary and grid value, at several magnitudes
    ties = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 4.0, 3.0, 2.0, 1.5, 1.0, 0.5, 0.125, 7.0])
    for s in (1.0, 1.0 / 3.0, 0.1, 2.0 ** -20, 2.0 ** 20):
        r = base.clone(); r[:16] = ties * s; rows.append(r)
        r = base.clone(); r[:16] = -ties * s; rows.append(r)
    # power-of-two ladder incl. the 2**(e-2) tie that bf16 data hits constantly
    r = base.clone(); r[:16] = 2.0 ** torch.arange(0, -16, -1, dtype=torch.float32); rows.append(r)
    r = base.clone(); r[:16] = 1.0 + 2.0 ** torch.arange(-1, -17, -1, dtype=torch.float32); rows.append(r)
    # tiny / huge
    r = base.clone(); r[0] = 2.0 ** -126; r[1] = 2.0 ** -130; r[2] = -(2.0 ** -140); rows.append(r)
    r = base.clone(); r[0] = 2.0 ** -120; r[1] = 2.0 ** -121; r[2] = 1.5 * 2.0 ** -122; rows.append(r)
    r = base.clone(); r[0] = 2.0 ** 100; r[1] = -3.0 * 2.0 ** 98; r[2] = 2.0 ** 97; rows.append(r)
    r = base.clone(); r[0] = 200.0; r[1] = 100.0; r[2] = -33.0; r[3] = 1.0; rows.append(r)   # NV scale near the top
    r = base.clone(); r[0] = 268.0; r[1] = 134.0; r[2] = -67.0; rows.append(r)
    r = base.clone(); r[0] = 1e-3; r[1] = 5e-4; r[2] = -2.5e-4; r[3] = 1e-5; rows.append(r)   # NV subnormal scales
    r = base.clone(); r[0] = 6e-4; r[1] = 5.9e-4; r[2] = 1e-4; rows.append(r)
    return torch.stack(rows)


def main(root: str) -> None:
    ref = _import_reference(root)
    torch.manual_seed(0)
    out: dict[str, np.ndarray] = {}

    # ---- rtn_e2m1 on a dense sweep incl. every tie -------------------------------
    sweep = torch.cat([torch.linspace(-7, 7, 1121, dtype=torch.float64),
                       torch.tensor([0.0, -0.0, 0.25, -0.25, 0.75, -0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -5.0, 1e-300, -1e-300],
                                    dtype=torch.float64)])
    sweep = sweep[: sweep.numel() // 2 * 2]
    vals, packed = ref.rtn_e2m1(sweep, mode="even", return_packed=True)
    out["e2m1_in"], out["e2m1_vals"], out["e2m1_packed"] = sweep.numpy(), vals.numpy(), _u8(packed)
    out["e2m1_unpacked"] = ref.unpack_e2m1(packed).numpy()

    # ---- rtn_xxfp4 / dequant_xxfp4 ------------------------------------------------
    g = torch.Generator().manual_seed(1234)
    for fmt, grp in (("mxfp4", 32), ("nvfp4", 16)):
        e = edge_inputs(grp)
        out[f"{fmt}_edge_in"] = e.numpy()
        for k, v in _quant(ref, e, fmt).items():
            out[f"{fmt}_edge_{k}"] = v
        x = torch.randn(48, 256, generator=g)
        x[:, 7] *= 50.0
        for tag, xi in (("f32", x), ("bf16", x.to(torch.bfloat16))):
            out[f"{fmt}_rand_{tag}_in"] = xi.to(torch.float64).numpy()
            for k, v in _quant(ref, xi, fmt).items():
                out[f"{fmt}_rand_{tag}_{k}"] = v

    # ---- fp8 scale casts as torch performs them -----------------------------------
    bits = torch.randint(0, 2 ** 31 - 1, (20000,), generator=g, dtype=torch.int64).to(torch.int32)
    f = bits.view(torch.float32)
    f = f[torch.isfinite(f)]
    f = torch.cat([f, torch.tensor([0.0, 2.0 ** -127, 2.0 ** -126, 1.5 * 2 ** -127, 0.75, 1.5, 3e38, 448.0, 464.0, 465.0, 480.0,
                                    2.0 ** -9, 1.5 * 2.0 ** -9, 2.0 ** -10, 2.0 ** -6, 0.9 * 2.0 ** -6])])
    out["cast_in"] = f.to(torch.float64).numpy()
    out["cast_e8m0"] = _u8(f.to(torch.float64).to(torch.float8_e8m0fnu))
    small = f[(f.abs() < 1e4)]
    out["cast_e4m3_in"] = small.to(torch.float64).numpy()
    out["cast_e4m3"] = _u8(small.to(torch.float64).to(torch.float8_e4m3fn))

    # ---- get_transform + block_transform ------------------------------------------
    for grp in (32, 16):
        c, r, tok = 4 * grp, 48, 64
        xc = torch.randn(tok, c, generator=g, dtype=torch.float64)
        xc[:, 3] *= 50.0
        h = xc.T @ xc / tok
        h += torch.eye(c, dtype=torch.float64) * 1e-2 * h.diagonal().mean()
        basis = torch.linalg.cholesky(h, upper=True)
        w = torch.randn(r, c, generator=g, dtype=torch.float64) * 0.02
        yfull = basis @ w.T
        ts = []
        for i in range(c // grp):
            sl = slice(i * grp, (i + 1) * grp)
            ts.append(ref.get_transform(basis=basis[sl, sl], y=yfull[sl], transform_type="wush",
                                        transform_dtype=torch.bfloat16))
            if i == 0:
                out[f"tf{grp}_hadamard"] = ref.get_transform(basis=basis[sl, sl], y=yfull[sl], transform_type="hadamard",
                                                             transform_dtype=torch.bfloat16).numpy()
        t = torch.stack(ts)
        out[f"tf{grp}_basis"], out[f"tf{grp}_y"], out[f"tf{grp}_wush"] = basis.numpy(), yfull.numpy(), t.numpy()
        xa = torch.randn(40, c, generator=g).to(torch.bfloat16)
        out[f"tf{grp}_x"] = xa.to(torch.float64).numpy()
        out[f"tf{grp}_bt_f32"] = ref.block_transform(xa.to(torch.float32), t).to(torch.float64).numpy()
        out[f"tf{grp}_bt_bf16"] = ref.block_transform(xa, t).to(torch.float64).numpy()
        fmt = "mxfp4" if grp == 32 else "nvfp4"
        for k, v in _quant(ref, ref.block_transform(xa.to(torch.float32), t), fmt).items():
            out[f"tf{grp}_q_{k}"] = v

    # ---- WUSH.update running mean (Triton launch replaced by the same fp32 product) ---
    xs = [torch.randn(1, 96, 64, generator=g).to(torch.bfloat16) for _ in range(3)]
    hess, n = torch.zeros(64, 64, dtype=torch.float32), 0
    for xi in xs:
        inp = xi.flatten(end_dim=-2)
        b = inp.size(0)
        hess *= n / (n + b)
        s = inp.to(torch.float32) * (n + b) ** -.5
        hess += s.T @ s
        n += b
    out["hess_in"] = torch.stack(xs).to(torch.float64).numpy()
    out["hess_out_f32"] = hess.numpy()

    np.savez_compressed(os.path.join(HERE, "reference_vectors.npz"), **out)
    print("wrote", os.path.join(HERE, "reference_vectors.npz"), {k: v.shape for k, v in out.items()})


def sweep_vectors(root: str) -> None:
    """Column sweep (gptq_babai_outer driven as quantize_layers drives it, wush_gptq.py:373-441) on
    small layers, both formats, three transforms, round-to-nearest and GPTQ, written to
    sweep_vectors.npz.  collate_xxfp4 cannot run on CPU (torch.cat of float4 tensors), so the blocks
    are collated here through uint8 views; everything else is the reference's code."""
    import functools
    ref = _import_reference(root)
    g = torch.Generator().manual_seed(4321)
    out: dict[str, np.ndarray] = {}
    for fmt, grp in (("mxfp4", 32), ("nvfp4", 16)):
        c, r, tok = 4 * grp, 40, 3 * grp
        xc = torch.randn(tok, c, generator=g, dtype=torch.float64)
        xc[:, 5] *= 50.0
        h = (xc.T @ xc / tok).to(torch.float32)
        w = (torch.randn(r, c, generator=g) * 0.02).to(torch.bfloat16)
        out[f"{fmt}_w"], out[f"{fmt}_h"] = w.to(torch.float64).numpy(), h.to(torch.float64).numpy()
        kw = dict(mxfp4=dict(group_size=32, scale_dtype=torch.float8_e8m0fnu, scale_scale=4., global_scale=3.),
                  nvfp4=dict(group_size=16, scale_dtype=torch.float8_e4m3fn, scale_scale=6., global_scale=10.))[fmt]
        quant_fn = functools.partial(ref.rtn_xxfp4, fp4_rounding_mode="even", **kw)
        for tt in ("identity", "hadamard", "wush"):
            for rtn in (True, False):
                collate = lambda *results, **_: results
                res = ref.gptq_babai_outer(
                    parameter=w, hessian=h,
                    inner_fn=functools.partial(
                        ref.block_transform_gptq_babai_inner, quant_fn=quant_fn,
                        basis_transform_fn=functools.partial(ref.get_transform, transform_type=tt,
                                                             transform_dtype=torch.bfloat16),
                        force_rtn_inner=rtn),
                    collate_fn=collate, block_size=grp, force_rtn_outer=rtn)
                tag = f"{fmt}_{tt}_{'rtn' if rtn else 'gptq'}"
                out[tag + "_e2m1"] = np.concatenate([_u8(x["e2m1"]) for x in res], axis=-1)
                out[tag + "_scale"] = np.concatenate([_u8(x["scale_quant"]) for x in res], axis=-1)
                out[tag + "_fake"] = torch.cat([ref.dequant_xxfp4(x["e2m1"], x["scale_quant"], x["global_scale"],
                                                                  dtype=torch.float64) for x in res], dim=-1).numpy()
                out[tag + "_transform"] = torch.stack([x["transform_basis"].to(torch.bfloat16).to(torch.float64)
                                                       for x in res]).numpy()
    np.savez_compressed(os.path.join(HERE, "sweep_vectors.npz"), **out)
    print("wrote", os.path.join(HERE, "sweep_vectors.npz"), {k: v.shape for k, v in out.items()})


def quest_vectors(root: str) -> None:
    """The reference's Triton pseudo-quantization kernel (inference_lib/src/fp_quant/module/triton/mxfp4.py) run on
    CPU by the Triton interpreter (TRITON_INTERPRET=1 must be set before this script starts), quest=True with the
    constant of pseudoquant_linear_fns.py:21 and, as a cross-check of the other branch, quest=False with 3/4.
    Inputs are float32 tensors holding bf16-representable values; transforms: identity and normalized Hadamard 32."""
    import importlib.util
    if os.environ.get("TRITON_INTERPRET") != "1":
        sys.exit("set TRITON_INTERPRET=1: the kernel has to run on CPU")
    spec = importlib.util.spec_from_file_location(
        "ref_triton_mxfp4", os.path.join(root, "inference_lib/src/fp_quant/module/triton/mxfp4.py"))
    mx = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mx)
    kernel = mx.mxfp4_forward_kernel.fn          # the function under the autotuner

    def run(x: torch.Tensor, had: torch.Tensor, quest: bool, gaussian_scale: float):
        x = x.contiguous()
        out = torch.empty_like(x)
        clip = torch.empty(x.shape, dtype=torch.bool)
        n = x.numel()
        kernel[((n + 1023) // 1024,)](x_ptr=x, hadamard_matrix_ptr=had.contiguous(), output_ptr=out, clip_mask_ptr=clip,
                                      n_elements=n, hadamard_dim=had.shape[0], group_size=32, gaussian_scale=gaussian_scale,
                                      quest=quest, WRITE_CLIP=True, BLOCK_SIZE=1024)
        return out.numpy().copy(), clip.numpy().copy()

    def sylvester(n: int) -> torch.Tensor:
        h = torch.tensor([[1.0]])
        while h.shape[0] < n:
            h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
        return h / n ** 0.5

    g = torch.Generator().manual_seed(777)
    bf = lambda t: t.to(torch.bfloat16).to(torch.float32)
    x = torch.randn(64, 128, generator=g)
    x[:, 7] *= 40.0                                   # an outlier channel: clipped under quest
    x[3] *= 1e-3
    x[5] *= 300.0
    x[8, :32] = 0.0                                   # an all-zero group
    x[9, :32] = 1.5                                   # a constant group: variance 0 up to rounding
    x[10, :32] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0] * 4) * torch.tensor([1.0, -1.0] * 16)
    x = bf(x)
    h = torch.tensor([[1.0]])
    while h.shape[0] < 32:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    had = bf(h / 32 ** 0.5)
    out = {"x": x.numpy(), "hadamard": had.numpy()}
    # transforms wider than the scale group: hadamard_group_size 64 and 128 (inference_lib/src/fp_quant/utils/config.py:44)
    had64, had128 = bf(sylvester(64)), bf(sylvester(128))
    out["hadamard64"], out["hadamard128"] = had64.numpy(), had128.numpy()
    for name, mat in (("identity", torch.eye(32)), ("hadamard", had), ("hadamard64", had64), ("hadamard128", had128)):
        for quest, gsc in ((True, 2.92247856 / 6.0), (False, 3.0 / 4.0)):
            o, c = run(x, mat, quest, gsc)
            tag = f"{name}_{'quest' if quest else 'absmax'}"
            out[tag + "_out"], out[tag + "_clip"] = o, c
    np.savez_compressed(os.path.join(HERE, "quest_vectors.npz"), **out)
    print("wrote", os.path.join(HERE, "quest_vectors.npz"), {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("WUSH_REFERENCE_ROOT")
    if not root:
        sys.exit("usage: make_golden.py <reference checkout> [sweep|quest]   (or set WUSH_REFERENCE_ROOT)")
    if len(sys.argv) > 2 and sys.argv[2] == "sweep":
        sweep_vectors(root)
    elif len(sys.argv) > 2 and sys.argv[2] == "quest":
        quest_vectors(root)
    else:
        main(root)
