"""The on-disk checkpoint format (wush_b200/checkpoint.py) without a GPU: shard splitting as the reference does it,
index and quantization_config contents, and a write -> read round trip of every tensor."""
import json
import os

import torch

from wush_b200 import checkpoint as ck


def _entries(n_layers=5, out=64, inp=128, g=32):
    gen = torch.Generator().manual_seed(0)
    state = {}
    for i in range(n_layers):
        state[f"model.layers.{i // 2}.mlp.proj{i}"] = {
            "qweight": torch.randint(0, 256, (out, inp // 2), generator=gen, dtype=torch.uint8),
            "scales": torch.randint(0, 256, (out, inp // g), generator=gen, dtype=torch.uint8),
            "forward_hadamard_matrix": torch.randn(g, inp, generator=gen).to(torch.bfloat16),
            "backward_hadamard_matrix": torch.randn(g, inp, generator=gen).to(torch.bfloat16),
            "weight_global_scale": torch.tensor([3.0]),
            "act_global_scale": torch.tensor([3.0]),
        }
    return state


def test_round_trip_and_layout(tmp_path):
    state = _entries()
    other = {"model.norm.weight": torch.ones(128, dtype=torch.bfloat16), "big": torch.zeros(5000, dtype=torch.float32)}
    wm = ck.export_quantized_model(str(tmp_path), state, other, {"hidden_size": 128}, hadamard_group_size=32,
                                   format="mxfp", transform_class="wush", max_shard_size=12000)
    files = sorted(f for f in os.listdir(tmp_path) if f.endswith(".safetensors"))
    n = len(files)
    assert n > 2 and files[0] == f"model-{'1'.zfill(len(str(n)))}-of-{n}.safetensors"
    index = json.load(open(tmp_path / ck.INDEX_NAME))
    assert index["metadata"] == {} and index["weight_map"] == wm
    assert wm["big"] != wm["model.norm.weight"]                  # a tensor over the limit sits in a shard of its own
    cfg = json.load(open(tmp_path / "config.json"))
    assert cfg["hidden_size"] == 128
    assert cfg["quantization_config"] == {
        "forward_dtype": "mxfp4", "backward_dtype": "bf16", "forward_method": "abs_max", "hadamard_group_size": 32,
        "modules_to_not_convert": ["lm_head"], "quant_method": "fp_quant", "store_master_weights": False,
        "pseudoquantization": False, "transform_init": "wush"}
    tensors, qcfg = ck.load_checkpoint(str(tmp_path))
    flat = ck.flatten_state(state, other)
    assert set(tensors) == set(flat)
    for k, v in flat.items():
        assert tensors[k].dtype == v.dtype and torch.equal(tensors[k], v), k
    some, _ = ck.load_checkpoint(str(tmp_path), ["model.layers.0.mlp.proj1.qweight"])
    assert list(some) == ["model.layers.0.mlp.proj1.qweight"]
    fcfg = ck.config_from_checkpoint(qcfg)
    assert fcfg.transform_init == "wush" and fcfg.hadamard_group_size == 32 and fcfg.forward_dtype.value == "mxfp4"


def test_shard_split_follows_the_reference_rule():
    t = lambda n: torch.zeros(n, dtype=torch.uint8)
    shards = ck.split_into_shards({"a": t(6), "b": t(6), "c": t(30), "d": t(3), "e": t(3)}, 10)
    assert [list(s) for s in shards] == [["a"], ["b"], ["c"], ["d", "e"]]
