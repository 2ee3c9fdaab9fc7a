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
    cleaned = {_clean(key) for key in packed_sd}     # pair `.alpha` with `.packed_weight` on the cleaned names
    for key, value in packed_sd.items():
        k = _clean(key)
        if k.endswith(".packed_weight"):
            tern.setdefault(k[: -len(".packed_weight")], {})["packed"] = value
        elif k.endswith(".alpha") and k[: -len(".alpha")] + ".packed_weight" in cleaned:
            tern.setdefault(k[: -len(".alpha")], {})["alpha"] = value
        else:
            plain[k] = value
    own = model.state_dict()
    with torch.no_grad():
        for k, v in plain.items():
            if k not in own:
                raise KeyError(f"load_packed_state_dict: unexpected key {k}")
            if v.numel() != own[k].numel():
                raise ValueError(f"load_packed_state_dict: {k} has {v.numel()} elements, the model expects {own[k].numel()}")
            own[k].copy_(v.to(own[k].dtype).reshape(own[k].shape))   # containers store 0-dim scalars as [1]
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
        # everything else the model owns (norms, router, embedding, lm_head, decay, buffers of the state dict)
        # must come from the file too: a silently kept constructor value would run, and be wrong
        absent = [k for k in own if k not in plain and k not in entries]
        if absent:
            raise KeyError(f"load_packed_state_dict: the file lacks {absent[:3]}{' ...' if len(absent) > 3 else ''}")
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


# ---------------------------------------------------------------------------------------------------
# .jarvis-tbin container (experiments/architecture_matrix/ternary_packed/jarvis_tbin_format.py:9-29):
#   [0..7] magic b"JTBIN01\0", [8..11] version (u32 = 1), [12..15] JSON length (u32), JSON manifest, payload.
#   Manifest entries: name, is_ternary, orig_shape, packed_shape, alpha, dtype ("uint8_packed" | "bfloat16"),
#   offset, length (relative to the payload start).  Ternary tensors are the weight_packing.py bytes.
# ---------------------------------------------------------------------------------------------------
TBIN_MAGIC = b"JTBIN01\x00"
TBIN_VERSION = 1
TBIN_TERNARY_TAGS = ("q_proj", "k_proj", "v_proj", "out_proj", "w1", "w2")


def read_tbin(path: str):
    """-> (packed state dict in the `<key>.packed_weight` / `<key>.alpha` form, manifest dict).
    Feed the first to load_packed_state_dict."""
    import json
    import struct

    with open(path, "rb") as fh:
        magic = fh.read(8)
        if magic != TBIN_MAGIC:
            raise ValueError(f"read_tbin: invalid magic header {magic!r}")
        version, meta_len = struct.unpack("<II", fh.read(8))
        if version != TBIN_VERSION:
            raise ValueError(f"read_tbin: unsupported version {version}")
        meta = json.loads(fh.read(meta_len).decode("utf-8"))
        payload = fh.read()
    out = {}
    for e in meta["tensors"]:
        raw = payload[e["offset"]: e["offset"] + e["length"]]
        if len(raw) != e["length"]:
            raise ValueError(f"read_tbin: truncated payload for {e['name']}")
        if e["is_ternary"]:
            if e["dtype"] != "uint8_packed":
                raise ValueError(f"read_tbin: ternary tensor {e['name']} has dtype {e['dtype']}")
            out[e["name"] + ".packed_weight"] = torch.frombuffer(bytearray(raw), dtype=torch.uint8).reshape(e["packed_shape"])
            out[e["name"] + ".alpha"] = torch.tensor(e["alpha"], dtype=torch.float32)
        else:
            if e["dtype"] != "bfloat16":
                raise ValueError(f"read_tbin: dense tensor {e['name']} has dtype {e['dtype']}")
            out[e["name"]] = torch.frombuffer(bytearray(raw), dtype=torch.int16).view(torch.bfloat16).reshape(e["orig_shape"])
    return out, meta


def write_tbin(state_dict: dict, path: str, extra_metadata: dict | None = None, device="cuda"):
    """Writes a model state dict as a .jarvis-tbin container (quantising + packing on the GPU)."""
    import json
    import struct
    import time

    manifest, buffers, offset = [], [], 0
    n_tern = n_dense = 0
    for name, t in state_dict.items():
        if t.dim() == 2 and any(tag in name for tag in TBIN_TERNARY_TAGS):
            p, alpha = ops.pack_ternary(t.detach().to(device=device, dtype=torch.float32).contiguous())
            raw = p.cpu().numpy().tobytes()
            entry = {"name": name, "is_ternary": True, "orig_shape": list(t.shape), "packed_shape": list(p.shape),
                     "alpha": float(alpha), "dtype": "uint8_packed"}
            n_tern += t.numel()
        else:
            raw = t.detach().cpu().to(torch.bfloat16).view(torch.int16).numpy().tobytes()
            entry = {"name": name, "is_ternary": False, "orig_shape": list(t.shape), "packed_shape": list(t.shape),
                     "alpha": 1.0, "dtype": "bfloat16"}
            n_dense += t.numel()
        entry.update(offset=offset, length=len(raw))
        manifest.append(entry)
        buffers.append(raw)
        offset += len(raw)
    meta = {"version": TBIN_VERSION, "format": "jarvis-tbin",
            "created_at": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()),
            "total_parameters": n_tern + n_dense, "ternary_parameters": n_tern, "dense_parameters": n_dense,
            "ternary_fraction_pct": 100.0 * n_tern / max(n_tern + n_dense, 1), "tensors": manifest,
            "extra": extra_metadata or {}}
    blob = json.dumps(meta).encode("utf-8")
    with open(path, "wb") as fh:
        fh.write(TBIN_MAGIC)
        fh.write(struct.pack("<II", TBIN_VERSION, len(blob)))
        fh.write(blob)
        for raw in buffers:
            fh.write(raw)
    return meta
