"""The reference's v1 GGUF-compatible container: the oracle's writer (a restatement
of save_gguf) against the package's reader on the CPU, and a Tiny-class checkpoint
loaded packed onto the GPU against the oracle's dense model over the decoded
tensors."""
import os
import struct

import numpy as np
import pytest

from oracle import gguf_writer as gw
from oracle import oracle as orc

CFG = dict(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn_hidden=512, vocab=512,
           max_seq=64, eps=1e-5, rope_theta=10000.0)


def _config_json(c, tied=True):
    return {"vocab_size": c["vocab"], "hidden_dim": c["d_model"], "ffn_dim": c["ffn_hidden"],
            "n_layers": c["n_layers"], "n_heads": c["n_heads"], "n_kv_heads": c["n_kv_heads"],
            "max_seq_len": c["max_seq"], "rope_theta": c["rope_theta"], "norm_eps": c["eps"],
            "tie_embeddings": tied}


def _tensors(c, seed=0):
    rng = np.random.default_rng(seed)
    qd, kd = c["n_heads"] * c["head_dim"], c["n_kv_heads"] * c["head_dim"]
    t = {"embedding.weight": rng.standard_normal((c["vocab"], c["d_model"])) * 0.02,
         "final_norm.weight": np.ones(c["d_model"])}
    for l in range(c["n_layers"]):
        t[f"blocks.{l}.norm1.weight"] = 0.75 + 0.001 * np.arange(c["d_model"])
        t[f"blocks.{l}.norm2.weight"] = np.ones(c["d_model"])
        for n, shp in {"attn.wq": (qd, c["d_model"]), "attn.wk": (kd, c["d_model"]), "attn.wv": (kd, c["d_model"]),
                       "attn.wo": (c["d_model"], qd), "ffn.w_gate": (c["ffn_hidden"], c["d_model"]),
                       "ffn.w_up": (c["ffn_hidden"], c["d_model"]), "ffn.w_down": (c["d_model"], c["ffn_hidden"])}.items():
            t[f"blocks.{l}.{n}.weight"] = rng.standard_normal(shp) * 0.02
    return {k: v.astype(np.float32) for k, v in t.items()}


def _reader():
    """The container parser alone: it needs neither a GPU nor the package's CUDA library."""
    import importlib.util
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    name = "ab2_gguf_format"
    if name not in sys.modules:
        spec = importlib.util.spec_from_file_location(name, os.path.join(root, "aarambh-ai_b200", "gguf_format.py"))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
    return sys.modules[name]


@pytest.mark.parametrize("fmt", ["q4_k_m", "q80"])
def test_container_round_trip_on_cpu(tmp_path, fmt):
    tensors = _tensors(CFG)
    path = str(tmp_path / "m.gguf")
    gw.save_gguf(path, _config_json(CFG), tensors, fmt)
    cfg, got_fmt, got, _keep = _reader().read_gguf(path)
    assert got_fmt == fmt and cfg["hidden_dim"] == CFG["d_model"]
    assert sorted(got) == sorted(tensors)
    for name, t in got.items():
        want = tensors[name]
        assert t.shape == want.shape
        if want.ndim == 1:
            assert t.encoding == gw.ENC_F32
            assert np.array_equal(np.frombuffer(t.payload, "<f4"), want)
        elif fmt == "q80":
            assert t.encoding == gw.ENC_Q8_0 and len(t.payload) == 4 + want.size
        else:
            assert t.encoding == gw.ENC_Q4KM and len(t.payload) == (want.size + 255) // 256 * 132
        # decode_tensor of the reference, restated, stays within the codec's error bound
        dec = gw.decode_tensor(t.encoding, t.shape, bytes(t.payload))
        assert dec.shape == want.shape
        assert np.abs(dec - want).max() <= (0.0 if want.ndim == 1 else 0.02)


def test_q4_payload_length_of_the_reference_known_answer():
    # (20, 15) ramp: payload = ceil(300 / 256) * 132 bytes and the decode keeps the shape (gguf.rs:324-338)
    t = (np.arange(300) * 0.01 - 1.5).astype(np.float32).reshape(20, 15)
    enc, payload = gw.encode_tensor("w", t, "q4_k_m")
    assert enc == gw.ENC_Q4KM and len(payload) == 2 * 132
    assert gw.decode_tensor(enc, t.shape, payload).shape == (20, 15)


def test_reader_rejects_bad_files(tmp_path):
    r = _reader()
    p = tmp_path / "bad.gguf"
    p.write_bytes(b"GGML" + b"\0" * 32)
    with pytest.raises(RuntimeError, match="not an Aarambh GGUF"):
        r.read_gguf(str(p))
    p.write_bytes(b"GGUF" + struct.pack("<I", 2) + b"\0" * 32)
    with pytest.raises(RuntimeError, match="unsupported GGUF version 2"):
        r.read_gguf(str(p))
    gw.save_gguf(str(p), _config_json(CFG), {"final_norm.weight": np.ones(8, np.float32)}, "q80")
    data = p.read_bytes()
    p.write_bytes(data[:-3])
    with pytest.raises(RuntimeError, match="truncated"):
        r.read_gguf(str(p))


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["q4_k_m", "q80"])
def test_checkpoint_loads_packed_and_matches_the_dense_oracle(tmp_path, fmt):
    import torch
    from helpers import pkg, rel_err
    p = pkg()
    tensors = _tensors(CFG)
    path = str(tmp_path / "m.gguf")
    gw.save_gguf(path, _config_json(CFG), tensors, fmt)
    model = p.gguf.load_gguf_model(path, dtype=torch.float32, max_tokens=32)
    # the reference's loader: decode every tensor to dense f32, then a dense model
    names = {"embedding.weight": "embedding", "final_norm.weight": "final_norm"}
    for l in range(CFG["n_layers"]):
        names[f"blocks.{l}.norm1.weight"] = f"layers.{l}.norm1"
        names[f"blocks.{l}.norm2.weight"] = f"layers.{l}.norm2"
        for w in ("wq", "wk", "wv", "wo"):
            names[f"blocks.{l}.attn.{w}.weight"] = f"layers.{l}.{w}"
        for w in ("w_gate", "w_up", "w_down"):
            names[f"blocks.{l}.ffn.{w}.weight"] = f"layers.{l}.{w}"
    dense = {}
    for name, value in tensors.items():
        enc, payload = gw.encode_tensor(name, value, fmt)
        dense[names[name]] = gw.decode_tensor(enc, value.shape, payload)
    dense["lm_head"] = dense["embedding"]
    cpu = orc.DenseModel(CFG, dense, 1, 32)
    ids = np.random.default_rng(3).integers(0, CFG["vocab"], 11)
    cache = model.empty_kv_cache_with_capacity(32)
    got = model.forward_with_cache(ids[None], 0, cache).float().cpu().numpy()
    ref = cpu.forward(ids[None], [0])
    assert rel_err(got, ref) < 1e-4
    # packed, not dense: the embedding table takes about a byte (q80) or half a byte per weight
    per_weight = model.weights["embedding"].nbytes() / tensors["embedding.weight"].size
    assert per_weight < (1.1 if fmt == "q80" else 0.6)
