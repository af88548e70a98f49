"""Data-parallel calibration and quantization of a model, block by block: the multi-GPU form of
``wush_quantization_gptq`` (src/quantization/wush_gptq.py:472-626), with the same signature and return values.

One process per GPU, every process holding a replica of the model.  What changes against the reference loop:
  * the calibration sequences are dealt to the ranks (rank r takes samples r, r + world, ...): every rank runs only
    its own sequences through a block, so the forward passes -- and the tokens every Hessian sums over -- are
    sharded;
  * the second moment of a layer input is accumulated by ``DistributedHessian`` (raw sums on the tensor cores, one
    combine over NVLink per matrix, the 1/N factor applied once) instead of the per-call rescaling of
    ``WUSH.update`` (:456-469);
  * layers that see the same input share ONE accumulator: q/k/v and gate/up hook the same tensor, so a block needs
    four second moments, not seven (the reference builds seven, three plus two of them identical, :511-534);
  * the column sweeps of a block's seven layers are dealt to the ranks too and the results broadcast, so the
    sweep -- the most expensive part -- also scales with the number of GPUs;
  * the block-output error that the reference prints (:564-576) is averaged over all ranks' sequences.
The quantized layers, the export dictionary (:584-601) and the hand-over of the quantized block's outputs to the next
block (:603-613) are as in the reference.

`hessian_factory`, `quantize_fn` and `layer_factory` exist so that the host logic can run on CPU ranks (gloo) with stand-ins for the
kernels; the defaults use the GPU kernels.
"""
from __future__ import annotations

import itertools
from typing import Callable, Optional

import torch
from torch import nn

LAYER_SEQUENCES = [
    ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"],
    ["self_attn.o_proj"],
    ["mlp.gate_proj", "mlp.up_proj"],
    ["mlp.down_proj"],
]


class ForwardInterrupt(Exception):
    pass


class InputCollector(nn.Module):
    """Stands in for the first block while the embeddings run: records the block's inputs and stops the forward
    pass (src/utils/model_utils.py:17-50)."""

    def __init__(self, module: nn.Module, cpu_offload: bool = False):
        super().__init__()
        self.module, self.cpu_offload = module, cpu_offload
        self.input_args, self.input_kwargs = [], []

    def forward(self, *args, **kwargs):
        if self.cpu_offload:
            args, kwargs = _to(args, device="cpu"), _to(kwargs, device="cpu")
        self.input_args.append(args)
        self.input_kwargs.append(kwargs)
        raise ForwardInterrupt

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self.module, name)


def _to(data, *a, **k):
    if isinstance(data, torch.Tensor):
        return data.to(*a, **k)
    if isinstance(data, (tuple, list)):
        return type(data)(_to(x, *a, **k) for x in data)
    if isinstance(data, dict):
        return {key: _to(v, *a, **k) for key, v in data.items()}
    return data


def _first(x):
    return x[0] if isinstance(x, (tuple, list)) else x


def _dist(group):
    import torch.distributed as dist
    on = dist.is_available() and dist.is_initialized()
    return dist, (dist.get_world_size(group) if on else 1), (dist.get_rank(group) if on else 0)


def _default_hessian_factory(hidden: int, device, group):
    from .hessian import DistributedHessian
    return DistributedHessian(hidden, device, group=group)


def _default_quantize(*weights, hessian, quant_type, transform_class, force_rtn):
    from .gptq import quantize_layers
    return quantize_layers(*weights, hessian=hessian, quant_type=quant_type, transform_class=transform_class,
                           force_rtn=force_rtn)


def _default_layer_factory(fake_weight: torch.Tensor, transform: torch.Tensor, quant_type: str):
    from .gptq import BlockTransformQuantizer, QuantLinear
    return QuantLinear(weight=fake_weight, activation_quantizer=BlockTransformQuantizer(transform=transform, quant_type=quant_type))


def _broadcast_layer(layer_and_result, weight: torch.Tensor, quant_type: str, src: int, rank: int, dist, group,
                     layer_factory):
    """Ship one quantized layer (pseudo-quantized weight, transforms, codes, scales) from the rank that swept it to
    all others; every rank -- the sender included -- rebuilds the layer from the shipped tensors, so all end with
    identical modules."""
    from .gptq import _FORMATS
    g = _FORMATS[quant_type]["group"]
    rows, cols = weight.shape
    dev, dt = weight.device, weight.dtype
    if rank == src:
        layer, res = layer_and_result
        fake = layer.weight.data.to(dt).contiguous()
        tb = res["transform_basis"].to(dt).contiguous()
        qw = res["qweight"].view(torch.uint8).contiguous()
        sc = res["scale_quant"].view(torch.uint8).contiguous()
    else:
        fake = torch.empty(rows, cols, dtype=dt, device=dev)
        tb = torch.empty(cols // g, g, g, dtype=dt, device=dev)
        qw = torch.empty(rows, cols // 2, dtype=torch.uint8, device=dev)
        sc = torch.empty(rows, cols // g, dtype=torch.uint8, device=dev)
    for t in (fake, tb, qw, sc):
        dist.broadcast(t, src=src, group=group)
    layer = layer_factory(fake, tb, quant_type).to(dev)
    res = {"transform_basis": tb, "qweight": qw, "scale_quant": sc.view(_FORMATS[quant_type]["scale_dtype"]),
           "global_scale": _FORMATS[quant_type]["global_scale"]}
    return layer, res


@torch.no_grad()
def wush_quantization_gptq(model, calibration_data, args, device, group=None, *, use_fused_layers: bool = False,
                           hessian_factory: Optional[Callable] = None, quantize_fn: Optional[Callable] = None,
                           layer_factory: Optional[Callable] = None, log: Callable = print):
    """(quantized_state_dict, non_quantized_state_dict), like the reference's function of the same name.

    model             a causal LM with `model.model.layers` (blocks whose linears are named as in LAYER_SEQUENCES) and
                      `get_input_embeddings()`; every rank passes an identical replica
    calibration_data  list of token-id tensors, the SAME list on every rank
    args              needs .format ('mxfp' | 'nvfp'), .gptq, .transform_class, .export_quantized_model,
                      .cpu_offload_activations, .cpu_offload_modules, .dtype
    use_fused_layers  quantize q/k/v (and gate/up) jointly with one transform per group of layers, the reference's
                      switch of the same name (:509-523, False there)
    """
    dist, world, rank = _dist(group)
    hessian_factory = hessian_factory or _default_hessian_factory
    quantize_fn = quantize_fn or _default_quantize
    layer_factory = layer_factory or _default_layer_factory
    quant_type = args.format + "4"
    quantized_state_dict, non_quantized_state_dict = {}, {}
    act_device = "cpu" if getattr(args, "cpu_offload_activations", False) else device
    offload_modules = getattr(args, "cpu_offload_modules", False)

    # ---- inputs of the first block, for this rank's share of the calibration sequences -----------------------
    blocks = model.model.layers
    blocks[0] = InputCollector(blocks[0], cpu_offload=getattr(args, "cpu_offload_activations", False))
    if offload_modules:
        model.get_input_embeddings().to(device)
        blocks[0] = blocks[0].to(device)
    for sample in calibration_data[rank::world]:
        try:
            model(sample.to(device=device))
        except ForwardInterrupt:
            pass
    input_args, input_kwargs = blocks[0].input_args, blocks[0].input_kwargs
    blocks[0] = blocks[0].module
    if offload_modules:
        model.get_input_embeddings().cpu()

    sequences = LAYER_SEQUENCES if use_fused_layers else [[n] for n in itertools.chain.from_iterable(LAYER_SEQUENCES)]
    input_of = {name: seq[0] for seq in LAYER_SEQUENCES for name in seq}      # layers that hook the same tensor

    for block_idx, block in enumerate(blocks):
        if rank == 0:
            log(f"Processing block {block_idx}...")
        if offload_modules:
            block.to(device)

        # ---- one second-moment accumulator per distinct layer input ------------------------------------------
        accumulators, hooks = {}, []
        for seq in LAYER_SEQUENCES:
            layer = block.get_submodule(seq[0])
            acc = accumulators[seq[0]] = hessian_factory(layer.weight.shape[1], layer.weight.device, group)

            def hook(_, inp, __, acc=acc):
                acc.update(inp[0])
            hooks.append(layer.register_forward_hook(hook))
        output_ref = []
        for a, k in zip(input_args, input_kwargs):
            out = block(*_to(a, device=device), **_to(k, device=device))
            output_ref.append(_first(out).to(act_device))
        for h in hooks:
            h.remove()
        hessians = {name: acc.finalize() for name, acc in accumulators.items()}    # the cross-rank combine

        # ---- column sweeps, dealt to the ranks ----------------------------------------------------------------
        force_rtn = not args.gptq
        quant_layers, real_results = {}, {}
        for i, seq in enumerate(sequences):
            weights = [block.get_submodule(n).weight for n in seq]
            owner = i % world
            mine = None
            if rank == owner:
                mine = quantize_fn(*weights, hessian=hessians[input_of[seq[0]]], quant_type=quant_type,
                                   transform_class=args.transform_class, force_rtn=force_rtn)
            for j, name in enumerate(seq):
                if world > 1:
                    payload = (mine[0][j], mine[1][j]) if mine is not None else None
                    quant_layers[name], real_results[name] = _broadcast_layer(payload, weights[j], quant_type, owner, rank,
                                                                              dist, group, layer_factory)
                else:
                    quant_layers[name], real_results[name] = mine[0][j], mine[1][j]
        for acc in accumulators.values():
            if hasattr(acc, "release"):
                acc.release()
        del hessians, accumulators

        # ---- swap the layers in, report the block-output error over all ranks' sequences ------------------------
        for name, layer in quant_layers.items():
            block.set_submodule(name, layer)
        losses = []
        for a, k, ref in zip(input_args, input_kwargs, output_ref):
            out = _first(block(*_to(a, device=device), **_to(k, device=device)))
            losses.append(torch.linalg.vector_norm(out - ref.to(out.device), dtype=torch.float32).pow(2.0) / ref.numel())
        stat = torch.stack([torch.stack(losses).sum() if losses else torch.zeros((), device=device),
                            torch.tensor(float(len(losses)), device=device)]).to(torch.float32)
        if world > 1:
            dist.all_reduce(stat, group=group)
        l2_loss = float(stat[0] / stat[1].clamp_min(1.0))
        if rank == 0:
            log(f"l2_loss block {block_idx}: {l2_loss}")

        # ---- export entries (wush_gptq.py:584-601) ---------------------------------------------------------------
        if getattr(args, "export_quantized_model", None):
            if args.export_quantized_model != "realquant":
                raise NotImplementedError("Only 'realquant' export is implemented.")
            cfg_dtype = getattr(getattr(model, "config", None), "torch_dtype", None) or torch.bfloat16
            orig_dtype = cfg_dtype if getattr(args, "dtype", "auto") == "auto" else args.dtype
            gs = 3.0 if args.format == "mxfp" else 10.0
            for name, layer in quant_layers.items():
                tm = layer.activation_quantizer.transform.to(dtype=orig_dtype).cpu()
                tm = tm.view(-1, tm.shape[-1]).T.contiguous()
                quantized_state_dict[f"model.layers.{block_idx}.{name}"] = {
                    "qweight": real_results[name]["qweight"].view(dtype=torch.uint8).cpu(),
                    "scales": real_results[name]["scale_quant"].view(torch.uint8).cpu(),
                    "forward_hadamard_matrix": tm,
                    "backward_hadamard_matrix": tm.clone(),
                    "weight_global_scale": torch.tensor([gs], dtype=torch.float32),
                    "act_global_scale": torch.tensor([gs], dtype=torch.float32),
                }

        # ---- the quantized block's outputs are the next block's inputs (:603-613) -----------------------------
        for a, k in zip(input_args, input_kwargs):
            out = _first(block(*_to(a, device=device), **_to(k, device=device))).to(act_device)
            if len(a) > 0:
                a[0].data = out
            elif "hidden_states" in k:
                k["hidden_states"] = out
            else:
                raise ValueError("Unsupported block input format.")
        if offload_modules:
            block.cpu()
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
    return quantized_state_dict, non_quantized_state_dict
