"""Checkpoint save / resume in the reference's binary format.

File layout (packages/train/src/checkpoint.ts:7-12, saveBinary :30-99, loadBinary :103-144):

    4 bytes   magic "ALPH"
    4 bytes   uint32 little-endian: byte length of the header
    N bytes   header, UTF-8 JSON: modelConfig, configHash, rngState, step,
              tokenizerArtifacts, optimizerStep, tensors = [{name, shape, elements}, ...]
    rest      the tensors' raw little-endian float32 data, concatenated in header order

Parameters come first as ``p.<name>`` in ``collectParamEntries`` order, then the optimizer
buffers as ``o.<name>.m`` / ``o.<name>.v`` with flat shapes (optimizers.ts:202-209).  The
legacy JSON form (a file that starts with "{", checkpoint.ts:160-186) is read as well.

What the device has to provide is only a coherent copy of the fp32 master parameters and of
the AdamW moments to the host (``TensorData.data`` synchronises and reads back) and the
upload on restore; the bf16 compute copies of the parameters are rebuilt from the restored
masters.
"""
from __future__ import annotations

import json
import os
import struct

import numpy as np

MAGIC = b"ALPH"


class CheckpointError(RuntimeError):
    """Mirrors CheckpointError of the reference (packages/core/src/errors.ts)."""


def save_checkpoint(path: str, state: dict) -> None:
    """state: {modelConfig, params: {name: ndarray}, optimizerState: {step, buffers: {name: ndarray}},
    rngState, configHash, step, tokenizerArtifacts?} (CheckpointState, checkpoint.ts:194-218)."""
    try:
        tensors, chunks = [], []
        for name, arr in state["params"].items():
            a = np.ascontiguousarray(arr, dtype="<f4")
            tensors.append({"name": f"p.{name}", "shape": [int(d) for d in np.shape(arr)], "elements": int(a.size)})
            chunks.append(a)
        opt = state.get("optimizerState") or {}
        for name, arr in (opt.get("buffers") or {}).items():
            a = np.ascontiguousarray(arr, dtype="<f4")
            tensors.append({"name": f"o.{name}", "shape": [int(d) for d in np.shape(arr)], "elements": int(a.size)})
            chunks.append(a)
        header = {
            "modelConfig": state.get("modelConfig"),
            "configHash": state.get("configHash"),
            "rngState": state.get("rngState"),
            "step": state.get("step"),
            "optimizerStep": int(opt.get("step", 0)),
            "tensors": tensors,
        }
        if state.get("tokenizerArtifacts") is not None:
            header["tokenizerArtifacts"] = state["tokenizerArtifacts"]
        hb = json.dumps(header, separators=(",", ":")).encode("utf-8")
        d = os.path.dirname(os.path.abspath(path))
        os.makedirs(d, exist_ok=True)
        tmp = path + ".tmp"
        with open(tmp, "wb") as f:
            f.write(MAGIC)
            f.write(struct.pack("<I", len(hb)))
            f.write(hb)
            for a in chunks:
                f.write(a.tobytes())
        os.replace(tmp, path)
    except Exception as e:  # the reference wraps every failure (checkpoint.ts:148-152)
        raise CheckpointError(f"Failed to save checkpoint: {e}") from e


def load_checkpoint(path: str) -> dict:
    try:
        with open(path, "rb") as f:
            raw = f.read()
        if raw[:4] == MAGIC:
            (hlen,) = struct.unpack_from("<I", raw, 4)
            header = json.loads(raw[8:8 + hlen].decode("utf-8"))
            off = 8 + hlen
            params, buffers = {}, {}
            for t in header["tensors"]:
                n = int(t["elements"])
                a = np.frombuffer(raw, dtype="<f4", count=n, offset=off).astype(np.float32).reshape(t["shape"])
                off += 4 * n
                if t["name"].startswith("p."):
                    params[t["name"][2:]] = a
                elif t["name"].startswith("o."):
                    buffers[t["name"][2:]] = a
            return {"modelConfig": header.get("modelConfig"), "params": params,
                    "optimizerState": {"step": int(header.get("optimizerStep") or 0), "buffers": buffers},
                    "tokenizerArtifacts": header.get("tokenizerArtifacts"), "rngState": header.get("rngState"),
                    "configHash": header.get("configHash"), "step": header.get("step")}
        parsed = json.loads(raw.decode("utf-8"))            # legacy JSON form
        params = {k: np.asarray(v["data"], dtype=np.float32).reshape(v["shape"]) for k, v in parsed["params"].items()}
        ob = (parsed.get("optimizerState") or {}).get("buffers") or {}
        buffers = {k: np.asarray(v["data"], dtype=np.float32).reshape(v["shape"]) for k, v in ob.items()}
        return {"modelConfig": parsed.get("modelConfig"), "params": params,
                "optimizerState": {"step": int((parsed.get("optimizerState") or {}).get("step", 0)), "buffers": buffers},
                "tokenizerArtifacts": parsed.get("tokenizerArtifacts"), "rngState": parsed.get("rngState"),
                "configHash": parsed.get("configHash"), "step": parsed.get("step")}
    except Exception as e:
        raise CheckpointError(f"Failed to load checkpoint: {e}") from e


def buildCheckpointState(trainer, rngState: int = 0, configHash: str = "", modelConfig=None,
                         tokenizerArtifacts=None) -> dict:
    """Host copy of a trainer's state (buildCheckpointState, checkpoint.ts:194-218): every
    parameter's fp32 master and the optimizer's moments are read back from the device."""
    mc = modelConfig if modelConfig is not None else dict(vars(trainer.mc))
    return {"modelConfig": mc, "params": trainer.host_params(), "optimizerState": trainer.opt.stateDict(),
            "tokenizerArtifacts": tokenizerArtifacts, "rngState": rngState, "configHash": configHash,
            "step": trainer.step_index}


def restoreParams(trainer, checkpointParams: dict) -> None:
    """restoreParams (checkpoint.ts:221-250): copy saved values into the existing parameters;
    a checkpoint with separate wq/wk/wv is packed into wqkv in that order."""
    for name, v in trainer.entries:
        saved = checkpointParams.get(name)
        if saved is None and name.endswith(".attn.wqkv"):
            prefix = name[:-len(".attn.wqkv")]
            parts = [checkpointParams.get(f"{prefix}.attn.{k}") for k in ("wq", "wk", "wv")]
            if all(p is not None for p in parts):
                saved = np.concatenate([np.asarray(p, dtype=np.float32).reshape(-1) for p in parts])
        if saved is None:
            continue
        arr = np.asarray(saved, dtype=np.float32).reshape(v.data.shape)
        trainer.load_param(name, arr)


def resume(trainer, state: dict) -> None:
    """Parameters, optimizer moments + step and the trainer's step counter from a loaded state."""
    restoreParams(trainer, state["params"])
    shapes = {n: tuple(v.data.shape) for n, v in trainer.entries}
    trainer.opt.loadStateDict(state["optimizerState"], shapes)
    trainer.step_index = int(state.get("step") or 0)
