"""Python face of tests/plain_ref.cpp, the second plain implementation (C++,
double precision, scalar loops).  Compiled with g++ on first use into a
temporary folder; called through ctypes with raw float64 arrays.  It shares no
code with tests/plain_llama.py nor with the engine."""
import ctypes
import hashlib
import os
import subprocess
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
_lib = None


def lib():
    global _lib
    if _lib is None:
        src = os.path.join(HERE, "plain_ref.cpp")
        tag = hashlib.sha256(open(src, "rb").read()).hexdigest()[:12]
        out = os.path.join(tempfile.gettempdir(), f"mdma_plain_ref_{os.getuid()}_{tag}.so")
        if not os.path.isfile(out):
            tmp = f"{out}.{os.getpid()}"
            subprocess.run(["g++", "-O2", "-shared", "-fPIC", "-std=c++17", src, "-o", tmp], check=True)
            os.replace(tmp, out)
        _lib = ctypes.CDLL(out)
    return _lib


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def ref_inv_freq(head_dim: int, theta: float, scaling) -> torch.Tensor:
    out = np.zeros(head_dim // 2, dtype=np.float64)
    s = scaling or {}
    lib().ref_inv_freq(ctypes.c_int(head_dim), ctypes.c_double(theta), ctypes.c_int(1 if scaling else 0),
                       ctypes.c_double(s.get("factor", 1.0)), ctypes.c_double(s.get("low_freq_factor", 1.0)),
                       ctypes.c_double(s.get("high_freq_factor", 1.0)),
                       ctypes.c_double(s.get("original_max_position_embeddings", 1.0)), _ptr(out))
    return torch.from_numpy(out)


def ref_forward(config: dict, tensors: dict, ids) -> torch.Tensor:
    """float64 logits [T, vocab] of one whole sequence."""
    L, E = config["num_hidden_layers"], config["hidden_size"]
    H = config["num_attention_heads"]
    K = config.get("num_key_value_heads") or H
    D = config.get("head_dim") or E // H
    F, V, T = config["intermediate_size"], config["vocab_size"], len(ids)
    tied = bool(config.get("tie_word_embeddings"))
    s = config.get("rope_scaling") or None
    layout = 0 if config.get("rope_layout", "split_half") == "interleaved" else 1
    sizes = np.asarray([L, E, H, K, D, F, V, T, layout, int(tied), 1 if s else 0], dtype=np.int32)
    s = s or {}
    reals = np.asarray([config["rms_norm_eps"], config.get("rope_theta", 10000.0), s.get("factor", 1.0),
                        s.get("low_freq_factor", 1.0), s.get("high_freq_factor", 1.0),
                        s.get("original_max_position_embeddings", 1.0)], dtype=np.float64)
    names = ["model.embed_tokens.weight"]
    for i in range(L):
        p = f"model.layers.{i}."
        names += [p + "input_layernorm.weight", p + "self_attn.q_proj.weight", p + "self_attn.k_proj.weight",
                  p + "self_attn.v_proj.weight", p + "self_attn.o_proj.weight", p + "post_attention_layernorm.weight",
                  p + "mlp.gate_proj.weight", p + "mlp.up_proj.weight", p + "mlp.down_proj.weight"]
    names += ["model.norm.weight", "model.embed_tokens.weight" if tied else "lm_head.weight"]
    arrays = [np.ascontiguousarray(tensors[n].to(torch.float64).numpy()) for n in names]
    ptrs = (ctypes.c_void_p * len(arrays))(*[a.ctypes.data for a in arrays])
    ids_a = np.asarray(list(ids), dtype=np.int32)
    logits = np.zeros((T, V), dtype=np.float64)
    lib().ref_forward(_ptr(sizes), _ptr(reals), ptrs, _ptr(ids_a), _ptr(logits))
    return torch.from_numpy(logits)
