"""MoE block of the engine's checkpoint file, from Python.

The engine's `weights.axiom` (writer core/src/training.cpp:283-392, loader
core/src/ai.cpp:273-491) holds no router or expert tensors.  The library appends
them as a tagged block after the transformer block (format in include/axm_moe.h);
these helpers call its host entry points with numpy arrays.  No GPU is needed.

    save_moe_block(path, weights, top_k)       weights: dict of fp32 arrays
    probe_moe_block(path) -> dict of sizes
    load_moe_block(path) -> (sizes, weights)
"""
import ctypes
import importlib
import os

import numpy as np

_pkg = importlib.import_module(__package__) if __package__ else None

NAMES = ("router_w", "router_bias", "w_gate", "w_up", "w_down", "shared_gate", "shared_up", "shared_down")


def _api():
    if _pkg is None:
        raise ImportError("import this module as part of its package")
    return _pkg


def _as_f32(a):
    if a is None:
        return None
    if hasattr(a, "detach"):  # a torch tensor on the host
        a = a.detach().float().cpu().numpy()
    return np.ascontiguousarray(a, dtype=np.float32)


def _table(arrays):
    api = _api()
    t = api.MoeCheckpoint()
    for n in NAMES:
        a = arrays.get(n)
        setattr(t, n, None if a is None else a.ctypes.data_as(ctypes.c_void_p))
    return t


def save_moe_block(path, weights, top_k):
    """Appends (or replaces) the MoE block of the existing checkpoint `path`.
    `weights`: router_w [D][E], w_gate / w_up [E][D][F], w_down [E][F][D], optionally
    router_bias [E] and shared_gate / shared_up [S][D][F], shared_down [S][F][D]."""
    api = _api()
    arrays = {n: _as_f32(weights.get(n)) for n in NAMES}
    D, E = arrays["router_w"].shape
    F = arrays["w_gate"].shape[2]
    S = 0 if arrays["shared_gate"] is None else arrays["shared_gate"].shape[0]
    expect = {"router_w": (D, E), "router_bias": (E,), "w_gate": (E, D, F), "w_up": (E, D, F),
              "w_down": (E, F, D), "shared_gate": (S, D, F), "shared_up": (S, D, F), "shared_down": (S, F, D)}
    for n, a in arrays.items():
        if a is not None and tuple(a.shape) != expect[n]:
            raise ValueError(f"{n} has shape {tuple(a.shape)}, expected {expect[n]}")
    desc = api.make_desc(0, D, F, E, top_k, S)
    table = _table(arrays)
    api.check(api.load().axm_moe_checkpoint_save(os.fsencode(path), ctypes.byref(desc), ctypes.byref(table)))


def probe_moe_block(path):
    api = _api()
    desc = api.make_desc(0, 0, 0, 0, 0)
    bias = ctypes.c_int32(0)
    api.check(api.load().axm_moe_checkpoint_probe(os.fsencode(path), ctypes.byref(desc), ctypes.byref(bias)))
    return {"d_model": desc.d_model, "d_ff": desc.d_ff, "num_experts": desc.num_experts, "top_k": desc.top_k,
            "num_shared": desc.num_shared, "router_bias": bool(bias.value)}


def load_moe_block(path):
    """Returns (sizes, weights): fp32 numpy arrays in the layouts of save_moe_block."""
    api = _api()
    info = probe_moe_block(path)
    D, F, E, S = info["d_model"], info["d_ff"], info["num_experts"], info["num_shared"]
    arrays = {"router_w": np.empty((D, E), np.float32), "router_bias": None,
              "w_gate": np.empty((E, D, F), np.float32), "w_up": np.empty((E, D, F), np.float32),
              "w_down": np.empty((E, F, D), np.float32),
              "shared_gate": None, "shared_up": None, "shared_down": None}
    if info["router_bias"]:
        arrays["router_bias"] = np.empty((E,), np.float32)
    if S:
        arrays["shared_gate"] = np.empty((S, D, F), np.float32)
        arrays["shared_up"] = np.empty((S, D, F), np.float32)
        arrays["shared_down"] = np.empty((S, F, D), np.float32)
    desc = api.make_desc(0, D, F, E, info["top_k"], S)
    table = _table(arrays)
    api.check(api.load().axm_moe_checkpoint_load(os.fsencode(path), ctypes.byref(desc), ctypes.byref(table)))
    return info, {n: a for n, a in arrays.items() if a is not None}
