"""Packed-checkpoint ingest and export (the data format on either side of the ternary layers).

Format of the reference's exporter (experiments/architecture_matrix/ternary_packed/
pack_model_checkpoint.py:52-94): every 2-D weight whose name contains one of the ternary-layer tags
is stored as `<key>.packed_weight` (uint8, runtime/weight_packing.py layout) plus `<key>.alpha`
(float32 scalar); everything else is stored as is (floating point in bf16); a leading `_orig_mod.`
is stripped from keys.  Loading installs the packed bytes and scales straight into the modules' GEMM
caches -- the fp32 master weight is filled with alpha * q for state-dict completeness, but is never
re-quantised (its own absmean would differ from the stored alpha).
"""
from __future__ import annotations

import torch

from . import ops
from .modules import AssociativeLinearAttention, SparseMoELayer, TernaryLinear

TERNARY_TAGS = ("q_proj", "k_proj", "v_proj", "out_proj", "w1", "w2", "w3", "gate_proj", "up_proj", "down_proj")


def _clean(key: str) -> str:
    return key[len("_orig_mod."):] if key.startswith("_orig_mod.") else key


def is_ternary_key(key: str, tensor: torch.Tensor) -> bool:
    return tensor.ndim == 2 and any(tag in key for tag in TERNARY_TAGS)


def export_packed_state_dict(state_dict: dict, device="cuda"):
    """fp32/bf16 state dict -> (packed state dict, metadata) in the reference exporter's format."""
    packed, meta = {}, {}
    for key, value in state_dict.items():
        k = _clean(key)
        if is_ternary_key(k, value):
            w = value.detach().to(device=device, dtype=torch.float32).contiguous()
            p, alpha = ops.pack_ternary(w)
            packed[f"{k}.packed_weight"] = p.cpu()
            packed[f"{k}.alpha"] = alpha.reshape(()).cpu()
            meta[k] = {"orig_shape": list(value.shape), "num_elements": value.numel(), "packed_bytes": p.numel(),
                       "alpha": float(alpha)}
        else:
            packed[k] = value.detach().to(torch.bfloat16).cpu() if value.is_floating_point() else value.detach().cpu()
    return packed, meta


def _install(cache, weights, packed_list, alpha_list, stack):
    canonical = torch.stack(packed_list) if stack else torch.cat(packed_list)
    cache.canonical = canonical
    cache.packed = ops.prepare_weights(canonical)
    cache.alpha = torch.stack([a.reshape(()) for a in alpha_list]).float()
    cache.key = tuple((w.data_ptr(), w._version, w.device) for w in weights)


def load_packed_state_dict(model: torch.nn.Module, packed_sd: dict) -> torch.nn.Module:
    """Loads a packed state dict into a (CUDA, eval) model built from jarvis_b200.modules."""
    dev = next(model.parameters()).device
    if dev.type != "cuda":
        raise RuntimeError("load_packed_state_dict: move the model to a CUDA device first")
    plain, tern = {}, {}
    for key, value in packed_sd.items():
        k = _clean(key)
        if k.endswith(".packed_weight"):
            tern.setdefault(k[: -len(".packed_weight")], {})["packed"] = value
        elif k.endswith(".alpha") and k[: -len(".alpha")] + ".packed_weight" in packed_sd:
            tern.setdefault(k[: -len(".alpha")], {})["alpha"] = value
        else:
            plain[k] = value
    own = model.state_dict()
    with torch.no_grad():
        for k, v in plain.items():
            if k not in own:
                raise KeyError(f"load_packed_state_dict: unexpected key {k}")
            own[k].copy_(v.to(own[k].dtype))
        entries = {}
        for k, d in tern.items():
            if k not in own:
                raise KeyError(f"load_packed_state_dict: unexpected key {k}")
            p = d["packed"].to(dev).contiguous()
            a = d["alpha"].to(dev, torch.float32).reshape(1)
            q = ops.unpack_ternary(p, own[k].shape, torch.float32)
            own[k].copy_(q * a)                                   # dequantised master weight
            entries[k] = (p, a)
        missing = [k for k, v in own.items() if is_ternary_key(k, v) and k not in entries]
        if missing:
            raise KeyError(f"load_packed_state_dict: missing packed weights for {missing[:3]} ...")
    mods = dict(model.named_modules())
    for name, mod in mods.items():
        pre = name + "." if name else ""
        if isinstance(mod, TernaryLinear):
            p, a = entries[pre + "weight"]
            _install(mod._cache, [mod.weight], [p], [a], stack=False)
        if isinstance(mod, AssociativeLinearAttention):
            trio = [entries[pre + f"{n}.weight"] for n in ("q_proj", "k_proj", "v_proj")]
            _install(mod._qkv, [mod.q_proj.weight, mod.k_proj.weight, mod.v_proj.weight], [t[0] for t in trio],
                     [t[1] for t in trio], stack=False)
        if isinstance(mod, SparseMoELayer):
            e1 = [entries[pre + f"w1.{e}.weight"] for e in range(mod.num_experts)]
            e2 = [entries[pre + f"w2.{e}.weight"] for e in range(mod.num_experts)]
            _install(mod._p1, [m.weight for m in mod.w1], [t[0] for t in e1], [t[1] for t in e1], stack=True)
            _install(mod._p2, [m.weight for m in mod.w2], [t[0] for t in e2], [t[1] for t in e2], stack=True)
    return model
