"""Host logic of the data-parallel calibration driver (wush_b200/calibrate.py) on 2 CPU ranks (gloo) with float32
stand-ins for the kernels: the calibration sequences are dealt to the ranks, layers that share an input share one
second moment (four per block), the second moments equal the single-process ones, the sweeps are dealt to the ranks
and their results broadcast (every rank ends with identical layers), and the export entries have the reference's
names and shapes.  Also: tile panels and token segments of the Hessian's overlapped combine."""
import os
import sys
import types

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch import nn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HID, FFN, VOCAB, SEQ, N_SAMPLES = 64, 96, 50, 12, 5


class _Attn(nn.Module):
    def __init__(self):
        super().__init__()
        self.q_proj, self.k_proj, self.v_proj, self.o_proj = (nn.Linear(HID, HID, bias=False) for _ in range(4))

    def forward(self, x):
        a = torch.softmax(self.q_proj(x) @ self.k_proj(x).transpose(-1, -2) / HID ** 0.5, dim=-1)
        return self.o_proj(a @ self.v_proj(x))


class _Mlp(nn.Module):
    def __init__(self):
        super().__init__()
        self.gate_proj, self.up_proj = nn.Linear(HID, FFN, bias=False), nn.Linear(HID, FFN, bias=False)
        self.down_proj = nn.Linear(FFN, HID, bias=False)

    def forward(self, x):
        return self.down_proj(torch.nn.functional.silu(self.gate_proj(x)) * self.up_proj(x))


class _Block(nn.Module):
    def __init__(self):
        super().__init__()
        self.self_attn, self.mlp = _Attn(), _Mlp()

    def forward(self, hidden_states):
        h = hidden_states + self.self_attn(hidden_states)
        return (h + self.mlp(h),)


class _Inner(nn.Module):
    def __init__(self):
        super().__init__()
        self.embed_tokens = nn.Embedding(VOCAB, HID)
        self.layers = nn.ModuleList([_Block(), _Block()])


class _Model(nn.Module):
    def __init__(self):
        super().__init__()
        self.model = _Inner()

    def get_input_embeddings(self):
        return self.model.embed_tokens

    def forward(self, ids):
        h = self.model.embed_tokens(ids)
        for blk in self.model.layers:
            h = blk(h)[0]
        return h


def _acc(h, x, r0, r1, lower_only, overwrite=False):
    xf = x.float()
    upd = xf[:, r0:r1].t() @ xf[:, :r1]
    rows, cols = torch.arange(r0, r1)[:, None], torch.arange(r1)[None, :]
    h[r0:r1, :r1] += torch.where(cols <= rows, upd, torch.zeros_like(upd))


def _fin(h, scale):
    low = torch.tril(h) * scale
    h.copy_(low + torch.tril(low, -1).t())


def _fake_quantize(*weights, hessian, quant_type, transform_class, force_rtn):
    """Stand-in for the GPU sweep: 'quantizes' by rounding to 1/64 and records which Hessian it was given."""
    from wush_b200.gptq import QuantLinear
    g = 32
    layers, results = [], []
    for w in weights:
        fake = (w.detach() * 64).round() / 64
        layers.append(QuantLinear(weight=fake, activation_quantizer=_Tagged(torch.eye(g).repeat(w.shape[1] // g, 1, 1), hessian)))
        results.append({"transform_basis": torch.eye(g).repeat(w.shape[1] // g, 1, 1),
                        "qweight": torch.zeros(w.shape[0], w.shape[1] // 2, dtype=torch.uint8),
                        "scale_quant": torch.full((w.shape[0], w.shape[1] // g), 127, dtype=torch.uint8).view(torch.float8_e8m0fnu),
                        "global_scale": 3.0})
    return layers, results


class _Tagged(nn.Module):
    def __init__(self, transform, hessian):
        super().__init__()
        self.register_buffer("transform", transform)
        self.hessian_trace = float(hessian.diagonal().sum())

    def forward(self, x):
        return x


def _args():
    return types.SimpleNamespace(format="mxfp", gptq=False, transform_class="wush", export_quantized_model="realquant",
                                 cpu_offload_activations=False, cpu_offload_modules=False, dtype=torch.float32)


def _data():
    g = torch.Generator().manual_seed(3)
    return [torch.randint(0, VOCAB, (1, SEQ), generator=g) for _ in range(N_SAMPLES)]


def _run(rank, world, port, out):
    sys.path.insert(0, ROOT)
    if world > 1:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
    from wush_b200 import calibrate
    from wush_b200.hessian import DistributedHessian
    torch.manual_seed(0)
    model = _Model()
    made = []

    def factory(hidden, device, group):
        dh = DistributedHessian(hidden, "cpu", group=group, accumulate_fn=_acc, finalize_fn=_fin)
        made.append(dh)
        return dh

    swept = []

    def quantize(*weights, **kw):
        swept.append(tuple(w.shape for w in weights))
        return _fake_quantize(*weights, **kw)

    from wush_b200.gptq import QuantLinear

    def layer_factory(fake, transform, quant_type):
        return QuantLinear(weight=fake, activation_quantizer=_Tagged(transform, torch.eye(2)))

    qsd, nq = calibrate.wush_quantization_gptq(model, _data(), _args(), "cpu", hessian_factory=factory, quantize_fn=quantize,
                                               layer_factory=layer_factory, log=lambda *_: None)
    traces = [float(dh.raw.diagonal().sum()) for dh in made]
    counts = [dh.num_samples for dh in made]
    state = {k: v.clone() for k, v in model.state_dict().items() if "weight" in k and "layers" in k}
    torch.save({"qsd": qsd, "traces": traces, "counts": counts, "swept": swept, "state": state,
                "local": [dh.local_tokens for dh in made]}, f"{out}.{rank}")
    if world > 1:
        dist.destroy_process_group()


def test_two_ranks_reproduce_the_single_process_run(tmp_path):
    one, two = str(tmp_path / "one"), str(tmp_path / "two")
    _run(0, 1, 0, one)
    mp.spawn(_run, args=(2, 29800 + os.getpid() % 500, two), nprocs=2, join=True)
    ref = torch.load(one + ".0", weights_only=False)
    r0, r1 = (torch.load(f"{two}.{r}", weights_only=False) for r in range(2))
    # four second moments per block (q/k/v and gate/up share theirs), two blocks
    assert len(ref["traces"]) == len(r0["traces"]) == 8
    # the tokens are sharded: 3 + 2 sequences, and the combined count is the whole calibration set
    assert r0["local"][0] == 3 * SEQ and r1["local"][0] == 2 * SEQ
    assert ref["counts"] == r0["counts"] == r1["counts"] == [N_SAMPLES * SEQ] * 8
    assert np.allclose(r0["traces"], ref["traces"], rtol=1e-5) and r0["traces"] == r1["traces"]
    # every rank sweeps only its share of the seven layers of a block, and all end with the same layers
    assert len(ref["swept"]) == 14 and len(r0["swept"]) == 8 and len(r1["swept"]) == 6
    for k in r0["state"]:
        assert torch.equal(r0["state"][k], r1["state"][k]), k
        assert torch.allclose(r0["state"][k], ref["state"][k], atol=1e-6), k
    names = {f"model.layers.{b}.{n}" for b in range(2) for n in ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj",
             "self_attn.o_proj", "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj")}
    assert set(ref["qsd"]) == set(r0["qsd"]) == names
    e = r0["qsd"]["model.layers.1.mlp.down_proj"]
    assert set(e) == {"qweight", "scales", "forward_hadamard_matrix", "backward_hadamard_matrix", "weight_global_scale",
                      "act_global_scale"}
    assert e["qweight"].shape == (HID, FFN // 2) and e["scales"].shape == (HID, FFN // 32)
    assert e["forward_hadamard_matrix"].shape == (32, FFN) and float(e["act_global_scale"]) == 3.0


def test_tile_panels_and_token_segments():
    from wush_b200.hessian import tile_panels, token_segments
    for n_tiles, per_wave in [(136, 74), (1596, 74), (10, 74), (148, 74), (223, 74), (75, 74), (1, 74), (0, 74)]:
        p = tile_panels(n_tiles, per_wave)
        assert (p[0][0] == 0 and p[-1][1] == n_tiles) if n_tiles else p == []
        assert all(a[1] == b[0] for a, b in zip(p, p[1:])) and all(b > a for a, b in p)
        assert all(a % per_wave == 0 for a, _ in p) and len(p) <= 7 + n_tiles // (3 * per_wave)
        assert all(b - a <= 3 * per_wave for a, b in p)             # short enough to be combined out of the L2
        assert len(tile_panels(n_tiles, per_wave, max_waves=0)) <= 7
        if n_tiles > per_wave:
            assert p[-1][1] - p[-1][0] <= per_wave              # only the last wave's combine is not hidden
    for tokens in (1, 32768, 49151, 49152, 65536, 262144, 70000):
        segs = token_segments(tokens)
        assert sum(n for _, n in segs) == tokens and all(a + n == b for (a, n), (b, _) in zip(segs, segs[1:]))
        assert all(n == 32768 for _, n in segs[:-1]) and segs[-1][1] < 49152
