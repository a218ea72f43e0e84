"""Checkpoints on disk: a directory of safetensors shards + `model.safetensors.index.json` + `config.json`, in
the serving weight formats (EXL3 trellis / MXFP4 + E8M0 / MXFP8 / FP8 128x128 block scaled / bf16), and the
loader that turns it into the nested weight dict the model runner takes -- whole, or as the shard of one
tensor/expert-parallel rank.

Layout of a tensor name: the path through the nested dict joined by dots, list indices as numbers, and for a packed
weight one entry per packed field, e.g. `layers.3.mix.in.trellis`, `layers.3.mix.in.suh`, `layers.3.mlp.w_gu.packed`.
The index file carries `weight_map` (name -> shard file), `weights` (non-tensor attributes of packed weights: codebook,
block sizes) and `structure` (the non-tensor leaves of the dict: layer types, flags).

Loading: every shard file is read through the C++ reader (header scan, offsets validated), tensors are memory-mapped
and cut to this rank's shard on the host WITHOUT decoding (`parallel.tp.shard_weights`: heads, intermediate columns,
experts by id, vocabulary rows), then each shard tensor goes to the device through pinned staging.  Expert stacks are
cut by index range, so a rank only ever touches the pages of its own experts.
Reference: engine-rs/src/weights.rs:194-283,627-818 (index scan, mmap, fast load, TP cuts), expert_load.rs:374-505
(expert arenas), ds41/load.rs:116-160, ds41/shard.rs:1-116 (pre-split shards: `write_rank_shards` below).
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from ..config import ModelConfig
from ..quant import formats as Q
from ..runtime import rt
from ..utils.safetensors_io import _DT, _RDT, write_safetensors

INDEX = "model.safetensors.index.json"


# ----------------------------------------------------------------------------- flatten / unflatten
def flatten(W) -> Tuple[Dict[str, torch.Tensor], dict, dict]:
    """(tensors by name, packed-weight attributes by weight name, non-tensor leaves by name)."""
    tensors, wmeta, structure = {}, {}, {}

    def rec(x, prefix):
        if isinstance(x, dict):
            structure[prefix + "{}"] = sorted(k for k in x)
            for k, v in x.items():
                rec(v, f"{prefix}{k}." if prefix or True else k)
        elif isinstance(x, list):
            structure[prefix + "[]"] = len(x)
            for i, v in enumerate(x):
                rec(v, f"{prefix}{i}.")
        elif isinstance(x, (torch.Tensor, Q.QuantWeight)):
            name = prefix[:-1]
            if isinstance(x, Q.Exl3Weight) and not x.experts and x.trellis._base is not None and name.endswith(("s_gu", "s_down")):
                structure[name] = "__view_of_stack__"          # the shared expert's views into the expert stacks
                return
            for field, t in Q.weight_tensors(x).items():
                tensors[f"{name}.{field}" if not isinstance(x, torch.Tensor) else name] = t
            if isinstance(x, Q.Exl3Weight):
                wmeta[name] = {"format": "exl3", "kind": x.kind, "bits": x.bits}
            elif isinstance(x, Q.Fp8BlockWeight):
                wmeta[name] = {"format": "fp8_block", "bn": x.bn, "bk": x.bk}
            elif isinstance(x, Q.Mxfp4Weight):
                wmeta[name] = {"format": "mxfp4"}
            elif isinstance(x, Q.Mxfp8Weight):
                wmeta[name] = {"format": "mxfp8"}
        else:
            structure[prefix[:-1]] = list(x) if isinstance(x, tuple) else x
    rec(W, "")
    return tensors, wmeta, structure


_FIELDS = ("trellis", "suh", "svh", "packed", "scales", "q8", "scales8", "q", "block_scales")


def unflatten(tensors: Dict[str, torch.Tensor], wmeta: dict, structure: dict):
    """Inverse of `flatten` (shared-expert views are rebuilt from the stacks)."""
    groups: Dict[str, dict] = {}
    for name, t in tensors.items():
        base, _, field = name.rpartition(".")
        if base in wmeta and field in _FIELDS:
            groups.setdefault(base, {})[field] = t
        else:
            groups[name] = t
    leaves = {}
    for name, g in groups.items():
        leaves[name] = Q.weight_from_tensors(g, wmeta[name]) if isinstance(g, dict) else g
    for name, v in structure.items():
        if not name.endswith(("{}", "[]")) and v != "__view_of_stack__":
            leaves[name] = tuple(v) if isinstance(v, list) else v

    def build(prefix):
        if prefix + "{}" in structure:
            out = {}
            for k in structure[prefix + "{}"]:
                name = f"{prefix}{k}"
                if structure.get(name) == "__view_of_stack__":
                    continue
                out[k] = build(name + ".") if (name + ".{}" in structure or name + ".[]" in structure) else leaves[name]
            return out
        n = structure[prefix + "[]"]
        return [build(f"{prefix}{i}.") for i in range(n)]
    W = build("")
    _rebuild_shared_views(W)
    return W


def _rebuild_shared_views(W):
    for lw in list(W.get("layers", [])) + list(W.get("mtp", {}).get("layers", [])):
        m = lw.get("mlp", {})
        if m.get("shared_in_stack"):
            e = m["w_gu"].trellis.shape[0] - 1
            for name, st in (("s_gu", m["w_gu"]), ("s_down", m["w_down"])):
                m[name] = Q.Exl3Weight(st.trellis[e], st.suh[e], st.svh[e], st.bits, st.kind)


# ----------------------------------------------------------------------------- save
def save_checkpoint(W: dict, cfg: ModelConfig, directory: str, max_shard_bytes: int = 4 << 30) -> None:
    os.makedirs(directory, exist_ok=True)
    tensors, wmeta, structure = flatten(W)
    shards, cur, size = [], {}, 0
    for name in sorted(tensors):
        t = tensors[name]
        n = t.numel() * t.element_size()
        if cur and size + n > max_shard_bytes:
            shards.append(cur)
            cur, size = {}, 0
        cur[name] = t
        size += n
    if cur:
        shards.append(cur)
    weight_map = {}
    for i, sh in enumerate(shards):
        fn = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        write_safetensors(os.path.join(directory, fn), sh, {"format": "spark_engine_b200"})
        for name in sh:
            weight_map[name] = fn
    with open(os.path.join(directory, INDEX), "w") as f:
        json.dump({"weight_map": weight_map, "weights": wmeta, "structure": structure}, f)
    with open(os.path.join(directory, "config.json"), "w") as f:
        f.write(cfg.to_json())


# ----------------------------------------------------------------------------- load
def _mapped_tensor(st, name: str) -> torch.Tensor:
    """Zero-copy host tensor over the file's pages (read-only mapping)."""
    info = st.info(name)
    n = info.end - info.begin
    dt = _RDT[info.dtype]
    if n == 0:
        return torch.empty(*info.shape, dtype=dt)
    mm = np.memmap(st.path(), dtype=np.uint8, mode="r", offset=st.data_offset() + info.begin, shape=(n,))
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")              # torch warns about non-writable arrays; the tensors are only read
        t = torch.from_numpy(mm)
    return t.view(dt).view(*info.shape)


def load_config(directory: str) -> ModelConfig:
    with open(os.path.join(directory, "config.json")) as f:
        return ModelConfig.from_dict(json.load(f))


def _to_device(x, device, pinned: bool):
    if isinstance(x, dict):
        return {k: _to_device(v, device, pinned) for k, v in x.items()}
    if isinstance(x, list):
        return [_to_device(v, device, pinned) for v in x]
    if isinstance(x, Q.QuantWeight):
        t = {k: _to_device(v, device, pinned) for k, v in Q.weight_tensors(x).items()}
        meta = {"kind": getattr(x, "kind", "mul1"), "bn": getattr(x, "bn", 128), "bk": getattr(x, "bk", 128)}
        return Q.weight_from_tensors(t, meta)
    if isinstance(x, torch.Tensor):
        if str(device) == "cpu":
            return x.clone() if not x.is_contiguous() or x._base is not None else x
        x = x.contiguous()
        if pinned and x.numel():
            stage = torch.empty(x.shape, dtype=x.dtype, pin_memory=True)
            stage.copy_(x)
            return stage.to(device, non_blocking=True)
        return x.to(device)
    return x


def _streamed_tensor(st, name: str, device) -> torch.Tensor:
    """A tensor read from its byte range of the file straight to `device` by the threaded loader (reader threads fill
    pinned staging buffers, copies are issued as they land; O_DIRECT with SPARK_LOAD_DIRECT=1): no mapping of the file,
    no second host copy.  Reference: engine-rs/src/weights.rs:194-283 (pread -> pinned staging -> device)."""
    from ..utils.devmem import load_file_range_to
    info = st.info(name)
    dt = _RDT[info.dtype]
    t = torch.empty(*info.shape, dtype=dt, device=device)
    if info.end > info.begin:
        load_file_range_to(t, st.path(), st.data_offset() + info.begin, chunk=32 << 20)
    return t


def load_checkpoint(directory: str, device="cpu", tp: Tuple[int, int] = (0, 1), pinned: bool = True,
                    cfg: Optional[ModelConfig] = None, stream: Optional[bool] = None):
    """-> (cfg, W) with W this rank's shard on `device`.  `stream` (default: SPARK_LOAD_STREAM=1): an unsharded load (one
    rank, or a directory written by `write_rank_shards`) reads every tensor straight to the device through the threaded
    loader instead of mapping the files."""
    cfg = cfg or load_config(directory)
    with open(os.path.join(directory, INDEX)) as f:
        idx = json.load(f)
    rank, world = tp
    if stream is None:
        stream = os.environ.get("SPARK_LOAD_STREAM", "0") == "1"
    stream = bool(stream) and world == 1
    files = {}
    tensors = {}
    for name, fn in idx["weight_map"].items():
        if fn not in files:
            files[fn] = rt().SafeTensors(os.path.join(directory, fn))        # validates the header and every offset
        tensors[name] = _streamed_tensor(files[fn], name, device) if stream else _mapped_tensor(files[fn], name)
    W = unflatten(tensors, idx["weights"], idx["structure"])
    if stream:
        _rebuild_shared_views(W)
        if str(device) != "cpu":
            torch.cuda.synchronize()
        return cfg, W
    if world > 1:
        from ..parallel.tp import shard_weights
        W = shard_weights(W, cfg, rank, world)
    W = _to_device(W, device, pinned and str(device) != "cpu" and torch.cuda.is_available())
    _rebuild_shared_views(W)
    if str(device) != "cpu":
        torch.cuda.synchronize()
    return cfg, W


def write_rank_shards(directory: str, out_root: str, world: int) -> None:
    """Pre-split a checkpoint into one directory per rank (`rank0`, `rank1`, ...), each a complete checkpoint of that
    rank's shard, so that start-up reads exactly the bytes a rank needs (ds41/shard.rs:1-116)."""
    cfg = load_config(directory)
    for r in range(world):
        _, Wr = load_checkpoint(directory, "cpu", tp=(r, world))
        save_checkpoint(Wr, cfg, os.path.join(out_root, f"rank{r}"))
