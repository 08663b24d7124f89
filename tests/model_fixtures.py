"""Builds the Tiny-class decoder of the benchmark spec on both sides: random
N(0, 0.02) weights (seed 0), quantised, as a GPU model over packed weights and as
the oracle's dense f32 model over the dequantised weights."""
import numpy as np
import torch

from helpers import pkg
from oracle import oracle as orc

TINY = dict(n_layers=6, d_model=384, n_heads=6, n_kv_heads=2, head_dim=64, ffn_hidden=1024, vocab=8192,
            max_seq=512, eps=1e-5, rope_theta=10000.0)
SMALL = dict(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn_hidden=512, vocab=512,
             max_seq=64, eps=1e-5, rope_theta=10000.0)


def shapes(c):
    qd, kd = c["n_heads"] * c["head_dim"], c["n_kv_heads"] * c["head_dim"]
    return {"wq": (qd, c["d_model"]), "wk": (kd, c["d_model"]), "wv": (kd, c["d_model"]),
            "wo": (c["d_model"], qd), "w_gate": (c["ffn_hidden"], c["d_model"]),
            "w_up": (c["ffn_hidden"], c["d_model"]), "w_down": (c["d_model"], c["ffn_hidden"])}


def random_weights(c, seed=0):
    rng = np.random.default_rng(seed)
    w = {"embedding": (rng.standard_normal((c["vocab"], c["d_model"])) * 0.02).astype(np.float32)}
    for l in range(c["n_layers"]):
        for name, shp in shapes(c).items():
            w[f"layers.{l}.{name}"] = (rng.standard_normal(shp) * 0.02).astype(np.float32)
        w[f"layers.{l}.norm1"] = np.ones(c["d_model"], np.float32)   # Init::Const(1.0)
        w[f"layers.{l}.norm2"] = np.ones(c["d_model"], np.float32)
    w["final_norm"] = np.ones(c["d_model"], np.float32)
    return w


def build_pair(c, method="int8_channel", dtype=torch.float32, seed=0, max_tokens=64, batch=1, capacity=160):
    """Returns (gpu_model, oracle_model, packed weights)."""
    p = pkg()
    dense = random_weights(c, seed)
    packed, deq = {}, {}
    for name, w in dense.items():
        if w.ndim == 2:
            lin = p.QuantLinear.quantise(torch.from_numpy(w).cuda(), method, 128)
            packed[name] = lin
            deq[name] = lin.dequantise().cpu().numpy()
        else:
            packed[name] = torch.from_numpy(w).cuda()
            deq[name] = w
    deq["lm_head"] = deq["embedding"]   # tied
    cfg = p.ModelConfig(c["n_layers"], c["d_model"], c["n_heads"], c["n_kv_heads"], c["head_dim"],
                        c["ffn_hidden"], c["vocab"], c["max_seq"], c["eps"], c["rope_theta"], True)
    gpu = p.AarambhModel(cfg, packed, dtype=dtype, max_tokens=max_tokens)
    cpu = orc.DenseModel(c, deq, batch, capacity)
    return gpu, cpu, packed
