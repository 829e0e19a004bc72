"""ctypes wrapper over the CPU oracle (oracle/libmoe_oracle.so).  Tests only."""
import ctypes
import os
import subprocess

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
LIB = os.path.join(ORACLE_DIR, "libmoe_oracle.so")


def _bf16_np(t):
    """torch bf16 tensor -> contiguous uint16 numpy view of its bits."""
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def _np_bf16(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


class Oracle:
    def __init__(self, lib):
        self.lib = lib
        vp, i32 = ctypes.c_void_p, ctypes.c_int
        lib.orc_num_threads.restype = ctypes.c_int
        lib.orc_router_logits.argtypes = [vp, vp, i32, vp, i32, i32, i32, vp]
        lib.orc_route_from_logits.argtypes = [vp, i32, i32, i32, vp, vp, vp, vp, vp]
        lib.orc_build_permutation.argtypes = [vp, i32, i32, i32, vp, vp, vp]
        lib.orc_aux_loss.argtypes = [vp, vp, i32, i32, i32, ctypes.c_float]
        lib.orc_aux_loss.restype = ctypes.c_float
        lib.orc_expert_ffn.argtypes = [vp, i32, i32, i32, vp, vp, vp, i32, vp]
        lib.orc_moe_backward.argtypes = [vp, vp, i32, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32,
                                         i32, ctypes.c_float, i32, vp, vp, vp, vp, vp, vp, vp]
        lib.orc_rmsnorm.argtypes = [vp, vp, i32, i32, ctypes.c_float, vp]
        lib.orc_set_threads.argtypes = [i32]
        lib.orc_adamw_engine.argtypes = ([vp] * 5 + [ctypes.c_int64, ctypes.c_int64] +
                                         [ctypes.c_float] * 5 + [ctypes.c_int64])
        lib.orc_moe_forward.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp,
                                        vp, vp, i32, i32, i32, i32, vp, vp]

    @staticmethod
    def _p(a):
        return None if a is None else a.ctypes.data_as(ctypes.c_void_p)

    def threads(self):
        return self.lib.orc_num_threads()

    def set_threads(self, n):
        self.lib.orc_set_threads(int(n))

    def adamw_engine(self, master, m, v, grad, w_bf16, in_dim, lr, b1, b2, eps, wd, step):
        """In place on the numpy arrays (fp32 master, m, v; uint16 bf16 copy)."""
        self.lib.orc_adamw_engine(self._p(master), self._p(m), self._p(v), self._p(grad),
                                  self._p(w_bf16), master.size, in_dim, lr, b1, b2, eps, wd, step)

    def router_logits(self, x, wr, bias=None):
        T, D = x.shape
        E = wr.shape[1]
        xb = _bf16_np(x)
        is32 = wr.dtype == torch.float32
        wn = wr.detach().cpu().contiguous().numpy() if is32 else _bf16_np(wr)
        bn = None if bias is None else bias.detach().cpu().contiguous().numpy().astype(np.float32)
        z = np.empty((T, E), dtype=np.float32)
        self.lib.orc_router_logits(self._p(xb), self._p(wn), int(is32), self._p(bn), T, D, E,
                                   self._p(z))
        return z

    def route(self, logits, k, counts=None):
        z = np.ascontiguousarray(logits, dtype=np.float32)
        T, E = z.shape
        idx = np.empty((T, k), dtype=np.int32)
        gates = np.empty((T, k), dtype=np.float32)
        probs = np.empty((T, E), dtype=np.float32)
        if counts is None:
            counts = np.zeros(E, dtype=np.int32)
        tie = np.zeros(T, dtype=np.uint8)
        self.lib.orc_route_from_logits(self._p(z), T, E, k, self._p(idx), self._p(gates),
                                       self._p(probs), self._p(counts), self._p(tie))
        return idx, gates, probs, counts, tie

    def permutation(self, idx, E):
        idx = np.ascontiguousarray(idx, dtype=np.int32)
        T, k = idx.shape
        offsets = np.empty(E + 1, dtype=np.int32)
        row_src = np.empty(T * k, dtype=np.int32)
        slot_dst = np.empty(T * k, dtype=np.int32)
        self.lib.orc_build_permutation(self._p(idx), T, E, k, self._p(offsets), self._p(row_src),
                                       self._p(slot_dst))
        return offsets, row_src, slot_dst

    def aux_loss(self, probs, idx, alpha):
        T, E = probs.shape
        return float(self.lib.orc_aux_loss(self._p(np.ascontiguousarray(probs)),
                                           self._p(np.ascontiguousarray(idx)), T, E, idx.shape[1],
                                           alpha))

    def rmsnorm(self, x, gamma, eps):
        T, D = x.shape
        y = np.empty((T, D), dtype=np.uint16)
        gn = None if gamma is None else gamma.detach().cpu().contiguous().numpy().astype(np.float32)
        self.lib.orc_rmsnorm(self._p(_bf16_np(x)), self._p(gn), T, D, eps, self._p(y))
        return _np_bf16(y).view(T, D)

    def expert_ffn(self, x_rows, wg, wu, wd, h_bf16=False):
        """One expert over the given bf16 rows: fp32 [n][D] numpy."""
        n, D = x_rows.shape
        F = wg.shape[1]
        o = np.zeros((n, D), dtype=np.float32)
        if n:
            self.lib.orc_expert_ffn(self._p(_bf16_np(x_rows)), n, D, F, self._p(_bf16_np(wg)),
                                    self._p(_bf16_np(wu)), self._p(_bf16_np(wd)), int(h_bf16),
                                    self._p(o))
        return o

    def backward(self, x, w, idx, gates, probs, dY, alpha=0.0, act_bf16=False, weight_grads=True):
        """Returns a dict of fp32 numpy gradients: dX, dWg, dWu, dWd, dWr, dgate, dlogits."""
        T, D = x.shape
        E, _, F = w["w_gate"].shape
        k = idx.shape[1]
        wr = w["router_w"]
        is32 = wr.dtype == torch.float32
        wn = wr.detach().cpu().contiguous().numpy() if is32 else _bf16_np(wr)
        out = {"dX": np.empty((T, D), np.float32), "dWr": np.empty((D, E), np.float32),
               "dgate": np.empty((T, k), np.float32), "dlogits": np.empty((T, E), np.float32)}
        if weight_grads:
            out.update({"dWg": np.empty((E, D, F), np.float32), "dWu": np.empty((E, D, F), np.float32),
                        "dWd": np.empty((E, F, D), np.float32)})
        g = lambda n: self._p(out[n]) if n in out else None
        self.lib.orc_moe_backward(
            self._p(_bf16_np(x)), self._p(wn), int(is32), self._p(_bf16_np(w["w_gate"])),
            self._p(_bf16_np(w["w_up"])), self._p(_bf16_np(w["w_down"])),
            self._p(np.ascontiguousarray(idx, dtype=np.int32)),
            self._p(np.ascontiguousarray(gates, dtype=np.float32)),
            self._p(np.ascontiguousarray(probs, dtype=np.float32)),
            self._p(np.ascontiguousarray(dY, dtype=np.float32)), T, D, E, k, F, alpha, int(act_bf16),
            g("dX"), g("dWg"), g("dWu"), g("dWd"), g("dWr"), g("dgate"), g("dlogits"))
        return out

    def forward(self, x, w, idx, gates, h_bf16=False, o_bf16=False, tok_range=None):
        """Returns (y, out) as torch bf16 [T][D]; rows outside tok_range are zero."""
        T, D = x.shape
        E, _, F = w["w_gate"].shape
        k = idx.shape[1]
        S = 0 if w.get("shared_gate") is None else w["shared_gate"].shape[0]
        xb = _bf16_np(x)
        wg, wu, wd = _bf16_np(w["w_gate"]), _bf16_np(w["w_up"]), _bf16_np(w["w_down"])
        sg = su = sd = None
        if S:
            sg, su, sd = (_bf16_np(w["shared_gate"]), _bf16_np(w["shared_up"]),
                          _bf16_np(w["shared_down"]))
        lo, hi = (0, T) if tok_range is None else tok_range
        y = np.zeros((T, D), dtype=np.uint16)
        out = np.zeros((T, D), dtype=np.uint16)
        idx = np.ascontiguousarray(idx, dtype=np.int32)
        gates = np.ascontiguousarray(gates, dtype=np.float32)
        self.lib.orc_moe_forward(self._p(xb), self._p(wg), self._p(wu), self._p(wd), self._p(idx),
                                 self._p(gates), T, D, E, k, F, S, self._p(sg), self._p(su),
                                 self._p(sd), int(h_bf16), int(o_bf16), lo, hi, self._p(y),
                                 self._p(out))
        return _np_bf16(y).view(T, D), _np_bf16(out).view(T, D)


_oracle = None


def load():
    global _oracle
    if _oracle is None:
        src = os.path.join(ORACLE_DIR, "moe_oracle.c")
        if not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(src):
            subprocess.run(["make", "-C", ORACLE_DIR], check=True, capture_output=True)
        _oracle = Oracle(ctypes.CDLL(LIB))
    return _oracle
