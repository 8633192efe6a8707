"""Checkpoint format and resume (packages/train/src/checkpoint.ts).  The byte layout is
pinned by a file assembled here with struct.pack from the layout the reference documents,
independently of the writer under test."""
import json
import struct

import numpy as np
import pytest

from alpha2_b200.checkpoint import (MAGIC, CheckpointError, buildCheckpointState, load_checkpoint, resume,
                                    save_checkpoint)


def _hand_made(path):
    w = np.arange(6, dtype="<f4").reshape(2, 3) * 0.5
    m = np.array([1.0, -2.0, 3.0, 0.0, 0.25, 8.0], dtype="<f4")
    header = {"modelConfig": {"vocabSize": 7}, "configHash": "abc", "rngState": 99, "step": 12, "optimizerStep": 12,
              "tensors": [{"name": "p.layer.0.attn.wo", "shape": [2, 3], "elements": 6},
                          {"name": "o.layer.0.attn.wo.m", "shape": [6], "elements": 6}]}
    hb = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(b"ALPH" + struct.pack("<I", len(hb)) + hb + w.tobytes() + m.tobytes())
    return w, m


def test_reads_the_reference_layout(tmp_path):
    w, m = _hand_made(tmp_path / "c.bin")
    st = load_checkpoint(str(tmp_path / "c.bin"))
    assert st["step"] == 12 and st["rngState"] == 99 and st["configHash"] == "abc"
    assert st["optimizerState"]["step"] == 12
    assert np.array_equal(st["params"]["layer.0.attn.wo"], w) and st["params"]["layer.0.attn.wo"].shape == (2, 3)
    assert np.array_equal(st["optimizerState"]["buffers"]["layer.0.attn.wo.m"], m)


def test_writer_produces_the_reference_layout(tmp_path):
    state = {"modelConfig": {"nLayer": 1}, "params": {"wte": np.array([[1.5, 2.5]], np.float32)},
             "optimizerState": {"step": 3, "buffers": {"wte.m": np.array([0.5, 0.25], np.float32),
                                                       "wte.v": np.array([4.0, 9.0], np.float32)}},
             "rngState": 5, "configHash": "h", "step": 3}
    p = tmp_path / "d" / "x.bin"
    save_checkpoint(str(p), state)
    raw = p.read_bytes()
    assert raw[:4] == MAGIC
    (hlen,) = struct.unpack_from("<I", raw, 4)
    header = json.loads(raw[8:8 + hlen])
    assert [t["name"] for t in header["tensors"]] == ["p.wte", "o.wte.m", "o.wte.v"]
    assert header["tensors"][0] == {"name": "p.wte", "shape": [1, 2], "elements": 2}
    assert header["optimizerStep"] == 3 and header["step"] == 3
    body = np.frombuffer(raw[8 + hlen:], dtype="<f4")
    assert body.tolist() == [1.5, 2.5, 0.5, 0.25, 4.0, 9.0]
    back = load_checkpoint(str(p))
    assert np.array_equal(back["params"]["wte"], state["params"]["wte"])


def test_legacy_json_and_errors(tmp_path):
    p = tmp_path / "old.json"
    p.write_text(json.dumps({"modelConfig": {}, "params": {"w": {"shape": [2], "data": [1, 2]}},
                             "optimizerState": {"step": 4, "buffers": {"w.m": {"shape": [2], "data": [3, 4]}}},
                             "rngState": 1, "configHash": "", "step": 4}))
    st = load_checkpoint(str(p))
    assert st["params"]["w"].tolist() == [1.0, 2.0] and st["optimizerState"]["buffers"]["w.m"].tolist() == [3.0, 4.0]
    with pytest.raises(CheckpointError):
        load_checkpoint(str(tmp_path / "missing.bin"))


def _trainer(backend, compute="f32"):
    from alpha2_b200.gpt import ModelConfig
    from alpha2_b200.trainer import TrainConfig, Trainer
    mc = ModelConfig(vocabSize=64, blockSize=16, nLayer=2, nEmbd=32, nHead=2, tied=True, init="plain",
                     compute_dtype=compute)
    return Trainer(backend, mc, TrainConfig(iters=10, batchSize=2, gradClip=0.5, seed=3))


def _steps(tr, batches, T):
    return [tr.train_step([(T(t, "i32"), T(g, "i32"))])["loss"] for t, g in batches]


def test_resume_matches_uninterrupted_run_on_the_host_backend(tmp_path):
    """4 steps == 2 steps + save + load into a fresh trainer + 2 steps, bit for bit
    (the reference's resume contract: parameters, moments, optimizer step, trainer step)."""
    from alpha2_b200.data import uniform_batches
    from tests.fake_backend import NumpyBackend, T
    batches = uniform_batches(7, 4, 2, 16, 64)
    a = _trainer(NumpyBackend())
    la = _steps(a, batches, T)
    b = _trainer(NumpyBackend())
    lb = _steps(b, batches[:2], T)
    save_checkpoint(str(tmp_path / "ck.bin"), buildCheckpointState(b, rngState=3))
    c = _trainer(NumpyBackend())
    resume(c, load_checkpoint(str(tmp_path / "ck.bin")))
    assert c.step_index == 2
    lc = _steps(c, batches[2:], T)
    assert la == lb + lc
    for (n, va), (_, vc) in zip(a.entries, c.entries):
        assert np.array_equal(va.data.data, vc.data.data), n


@pytest.mark.gpu
@pytest.mark.parametrize("compute", ["f32", "bf16"])
def test_resume_matches_uninterrupted_run_on_the_device(tmp_path, compute):
    from alpha2_b200.backend import CudaBackend
    from alpha2_b200.data import uniform_batches
    B = CudaBackend(0)
    up = lambda a, d: B.upload(a, d)
    batches = uniform_batches(7, 4, 2, 16, 64)
    a = _trainer(B, compute)
    la = _steps(a, batches, up)
    b = _trainer(B, compute)
    lb = _steps(b, batches[:2], up)
    save_checkpoint(str(tmp_path / "ck.bin"), buildCheckpointState(b, rngState=3))
    c = _trainer(B, compute)
    resume(c, load_checkpoint(str(tmp_path / "ck.bin")))
    lc = _steps(c, batches[2:], up)
    assert la == lb + lc
    for (n, va), (_, vc) in zip(a.entries, c.entries):
        assert np.array_equal(np.asarray(va.data.data), np.asarray(vc.data.data)), n
