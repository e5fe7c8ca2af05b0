"""ctypes front end of the CPU oracle (oracle/oracle.c).

TEST INFRASTRUCTURE ONLY.  Nothing under `bullet_b200/` imports this package; it is loaded
by `tests/`, by `__graft_entry__.smoke()` and by the CPU-baseline legs of `bench.py`, always
as the checker or as the timed CPU baseline, never as part of the product path.

`Oracle("f32")` follows the reference's fp32 interpreter arithmetic; `Oracle("f64")` is the
same code in double precision, used as an arbiter when two fp32 results disagree.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
TENSORS = ("l0w", "l0b", "l0f", "l1w", "l1b", "l2w", "l2b", "l3w", "l3b")
_HP_ORDER = TENSORS  # order of the hyper-parameter table taken by orc_net_update


def build(force: bool = False) -> None:
    """Compile both oracle libraries with the Makefile beside this file."""
    if force:
        subprocess.check_call(["make", "-C", _HERE, "clean"], stdout=subprocess.DEVNULL)
    subprocess.check_call(["make", "-C", _HERE], stdout=subprocess.DEVNULL)


class _Tensors(ctypes.Structure):
    _fields_ = [("l0w", ctypes.c_void_p), ("l0b", ctypes.c_void_p), ("l0f", ctypes.c_void_p),
                ("lw", ctypes.c_void_p * 3), ("lb", ctypes.c_void_p * 3)]


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


class Oracle:
    def __init__(self, precision: str = "f32"):
        path = os.path.join(_HERE, f"liboracle_{precision}.so")
        if not os.path.exists(path):
            build()
        self.lib = ctypes.CDLL(path)
        self.real = np.float32 if precision == "f32" else np.float64
        self.creal = ctypes.c_float if precision == "f32" else ctypes.c_double
        assert self.lib.orc_real_bytes() == np.dtype(self.real).itemsize
        self.lib.orc_net_grad.restype = ctypes.c_int
        self.lib.orc_map_chess.restype = ctypes.c_int
        self.lib.orc_map_ataxx147.restype = ctypes.c_int

    # ------------------------------------------------------------------ helpers
    def _r(self, a):
        return np.ascontiguousarray(a, dtype=self.real)

    @staticmethod
    def _i(a):
        return np.ascontiguousarray(a, dtype=np.int32)

    def _scalar(self, v):
        """Scalars reach the reference's kernels as f32; the f64 arbiter gets the same rounded values."""
        return self.creal(float(np.float32(v)))

    def threads(self) -> int:
        return int(self.lib.orc_max_threads())

    # ---------------------------------------------------------------------- ops
    def sparse_matmul(self, W, idx, batch, rows, cols, stride, offset, nnz):
        W, idx = self._r(W), self._i(idx)
        out = np.zeros(batch * rows, dtype=self.real)
        self.lib.orc_sparse_matmul(_ptr(W), _ptr(idx), _ptr(out), batch, rows, cols, stride, offset, nnz)
        return out

    def sparse_matmul_bwd_multi(self, pairs, batch, rows, cols, stride, nnz):
        """pairs: list of (grad, indices, offset)"""
        n = len(pairs)
        gs = [self._r(p[0]) for p in pairs]
        ids = [self._i(p[1]) for p in pairs]
        garr = (ctypes.c_void_p * n)(*[g.ctypes.data for g in gs])
        iarr = (ctypes.c_void_p * n)(*[i.ctypes.data for i in ids])
        offs = (ctypes.c_int * n)(*[p[2] for p in pairs])
        out = np.zeros(stride * cols, dtype=self.real)
        self.lib.orc_sparse_matmul_bwd_multi(n, garr, iarr, offs, _ptr(out), batch, rows, cols, stride, nnz)
        return out

    def matmul(self, lhs, rhs, b, m, n, k, lhs_col_mjr, rhs_col_mjr, integer=False):
        dt = np.int32 if integer else self.real
        lhs, rhs = np.ascontiguousarray(lhs, dtype=dt), np.ascontiguousarray(rhs, dtype=dt)
        out = np.zeros(b * m * k, dtype=dt)
        fn = self.lib.orc_matmul_i32 if integer else self.lib.orc_matmul
        fn(_ptr(lhs), _ptr(rhs), _ptr(out), b, m, n, k, int(lhs_col_mjr), int(rhs_col_mjr))
        return out

    def _typed(self, name, integer):
        return getattr(self.lib, name + ("_i32" if integer else "")), (np.int32 if integer else self.real)

    def select(self, x, indices, batch, inner, divisor, integer=False):
        fn, dt = self._typed("orc_select", integer)
        x = np.ascontiguousarray(x, dtype=dt)
        out = np.zeros(batch * (inner // divisor), dtype=dt)
        fn(_ptr(x), _ptr(self._i(indices)), _ptr(out), batch, inner, divisor)
        return out

    def select_pad(self, x, indices, batch, inner, divisor, integer=False):
        fn, dt = self._typed("orc_select_pad", integer)
        x = np.ascontiguousarray(x, dtype=dt)
        out = np.full(batch * inner, 7, dtype=dt)
        fn(_ptr(x), _ptr(self._i(indices)), _ptr(out), batch, inner, divisor)
        return out

    def reduce_sum(self, x, outer, dimen, inner, integer=False):
        fn, dt = self._typed("orc_reduce_sum", integer)
        x = np.ascontiguousarray(x, dtype=dt)
        out = np.zeros(outer * inner, dtype=dt)
        fn(_ptr(x), _ptr(out), outer, dimen, inner)
        return out

    def broadcast(self, x, outer, inner, repeats, integer=False):
        fn, dt = self._typed("orc_broadcast", integer)
        x = np.ascontiguousarray(x, dtype=dt)
        out = np.zeros(outer * inner * repeats, dtype=dt)
        fn(_ptr(x), _ptr(out), outer, inner, repeats)
        return out

    def act_forward(self, act, x):
        x = self._r(x)
        y = np.zeros_like(x)
        self.lib.orc_act_forward(act, _ptr(x), _ptr(y), x.size)
        return y

    def act_backward(self, act, y, gy):
        y, gy = self._r(y), self._r(gy)
        gx = np.zeros_like(y)
        self.lib.orc_act_backward(act, _ptr(y), _ptr(gy), _ptr(gx), y.size)
        return gx

    def adamw(self, p, m, v, g, adj, rate, hp):
        """In place on p, m, v (arrays of this oracle's precision)."""
        c = self._scalar
        self.lib.orc_adamw(_ptr(p), _ptr(m), _ptr(v), _ptr(g), ctypes.c_size_t(p.size), c(adj), c(rate),
                           c(hp.decay), c(hp.beta1), c(hp.beta2), c(hp.min_weight), c(hp.max_weight))

    def radam_step(self, step: int, beta1: float, beta2: float, threshold: float = 5.0):
        """(step size, use_denom) of RAdam's host-side schedule (radam.rs:295-314), in f32."""
        flag = ctypes.c_int()
        self.lib.orc_radam_step.restype = ctypes.c_float
        size = self.lib.orc_radam_step(step, ctypes.c_float(beta1), ctypes.c_float(beta2), ctypes.c_float(threshold), ctypes.byref(flag))
        return float(size), int(flag.value)

    def radam(self, p, m, v, g, adj, rate, use_denom, hp):
        """In place; `rate` = learning rate x step size (f32 product), hp with decay/beta1/beta2/min_weight/max_weight."""
        c = self._scalar
        self.lib.orc_radam(_ptr(p), _ptr(m), _ptr(v), _ptr(g), ctypes.c_size_t(p.size), c(adj), c(rate), int(use_denom),
                           c(hp.decay), c(hp.beta1), c(hp.beta2), c(hp.min_weight), c(hp.max_weight))

    def lookahead(self, w, slow, alpha):
        self.lib.orc_lookahead(_ptr(w), _ptr(slow), ctypes.c_size_t(w.size), self._scalar(alpha))

    def train_radam(self, desc, weights, batches, lr, params, ranger=None):
        """RAdam (or, with `ranger` = (alpha, k), Ranger) steps over `batches`, every tensor with the same
        parameters: -> (weights, m, v, slow or None, [loss_sum per step])."""
        w = self.to_real(weights)
        m, v = self.zeros_like(desc), self.zeros_like(desc)
        slow = self.zeros_like(desc) if ranger else None
        losses = []
        for step, (stm, nstm, buckets, targets) in enumerate(batches, start=1):
            loss, g, _ = self.net_grad(desc, w, stm, nstm, buckets, targets)
            size, use_denom = self.radam_step(step, params.beta1, params.beta2)
            rate = float(np.float32(lr) * np.float32(size))
            for k in w:
                self.radam(w[k], m[k], v[k], g[k], 1.0 / len(targets), rate, use_denom, params)
            if ranger and step % ranger[1] == 0:
                for k in w:
                    self.lookahead(w[k], slow[k], ranger[0])
            losses.append(loss)
        return w, m, v, slow, losses

    # -------------------------------------------------------------- featurisers
    def map_chess(self, records, nnz=32, layout32=None):
        n = len(records)
        stm = np.zeros((n, nnz), dtype=np.int32)
        ntm = np.zeros((n, nnz), dtype=np.int32)
        lay = self._i(layout32) if layout32 is not None else None
        rc = self.lib.orc_map_chess(_ptr(records), n, 0 if lay is None else 1,
                                    _ptr(lay) if lay is not None else None, _ptr(stm), _ptr(ntm), nnz)
        if rc < 0:
            raise ValueError("a record holds more features than nnz")
        return stm, ntm

    def map_ataxx147(self, records, nnz=49):
        n = len(records)
        stm = np.zeros((n, nnz), dtype=np.int32)
        ntm = np.zeros((n, nnz), dtype=np.int32)
        if self.lib.orc_map_ataxx147(_ptr(records), n, _ptr(stm), _ptr(ntm), nnz) < 0:
            raise ValueError("a record holds more features than nnz")
        return stm, ntm

    def material_count(self, records, nbuckets):
        out = np.zeros(len(records), dtype=np.int32)
        self.lib.orc_material_count(_ptr(records), len(records), nbuckets, _ptr(out))
        return out

    def make_targets(self, records, scale=400.0, blend=0.5):
        out = np.zeros(len(records), dtype=np.float32)
        dt = records.dtype
        self.lib.orc_make_targets(_ptr(records), len(records), dt.itemsize, dt.fields["score"][1],
                                  dt.fields["result"][1], ctypes.c_float(scale), ctypes.c_float(blend), _ptr(out))
        return out

    def map_batch(self, game, records, desc):
        """Reference-layout batch for one of the benchmark games: stm, nstm, buckets, targets."""
        from bullet_b200.configs import KING_BUCKETS_16  # plain data, no product code path

        if game == "chess768":
            stm, ntm = self.map_chess(records, desc.nnz)
        elif game == "chess_buckets":
            stm, ntm = self.map_chess(records, desc.nnz, KING_BUCKETS_16)
        elif game == "ataxx147":
            stm, ntm = self.map_ataxx147(records, desc.nnz)
        else:
            raise ValueError(game)
        if desc.n_out_buckets > 1:
            buckets = self.material_count(records, desc.n_out_buckets)
        else:
            buckets = np.zeros(len(records), dtype=np.int32)
        return stm, ntm, buckets, self.make_targets(records)

    # ---------------------------------------------------------------- whole net
    def _pack(self, desc, tensors):
        """dict name -> array  =>  (struct, keep-alive list of converted arrays, dict of them)"""
        s = _Tensors()
        conv = {}
        shapes = desc.tensor_shapes()
        for name in shapes:
            conv[name] = tensors[name] if (tensors[name].dtype == self.real and tensors[name].flags.c_contiguous) \
                else self._r(tensors[name])
            assert conv[name].size == shapes[name][0] * shapes[name][1], name
        s.l0w, s.l0b = conv["l0w"].ctypes.data, conv["l0b"].ctypes.data
        s.l0f = conv["l0f"].ctypes.data if "l0f" in conv else None
        for i in range(desc.n_dense):
            s.lw[i] = conv[f"l{i + 1}w"].ctypes.data
            s.lb[i] = conv[f"l{i + 1}b"].ctypes.data
        return s, conv

    def zeros_like(self, desc):
        return {k: np.zeros(r * c, dtype=self.real) for k, (r, c) in desc.tensor_shapes().items()}

    def to_real(self, tensors):
        return {k: np.array(v, dtype=self.real) for k, v in tensors.items()}

    def net_grad(self, desc, tensors, stm, nstm, buckets, targets, want_grads=True):
        """-> (loss_sum, grads dict or None, outputs[B])"""
        from bullet_b200.configs import CNetDesc

        cdesc = CNetDesc.from_desc(desc)
        B = len(targets)
        stm, nstm, buckets = self._i(stm), self._i(nstm), self._i(buckets)
        targets = np.ascontiguousarray(targets, dtype=np.float32)
        ws, keep = self._pack(desc, tensors)
        grads = self.zeros_like(desc) if want_grads else None
        gs, gkeep = self._pack(desc, grads) if want_grads else (None, None)
        loss = self.creal(0)
        out = np.zeros(B, dtype=self.real)
        rc = self.lib.orc_net_grad(ctypes.byref(cdesc), ctypes.byref(ws), _ptr(stm), _ptr(nstm), _ptr(buckets),
                                   _ptr(targets), B, ctypes.byref(gs) if want_grads else None, ctypes.byref(loss),
                                   _ptr(out))
        if rc != 0:
            raise ValueError("oracle rejected the network description")
        return float(loss.value), grads, out

    def net_update(self, desc, weights, m, v, grads, adj, rate, hp):
        """In place AdamW on dicts of arrays of this oracle's precision; hp: dict name -> AdamWParams."""
        cdesc = None
        from bullet_b200.configs import CNetDesc

        cdesc = CNetDesc.from_desc(desc)

        class HP(ctypes.Structure):
            _fields_ = [(n, self.creal) for n in ("decay", "beta1", "beta2", "wmin", "wmax")]

        table = (HP * 9)()
        for i, name in enumerate(_HP_ORDER):
            p = hp[name] if isinstance(hp, dict) else hp
            table[i] = HP(*[float(np.float32(x)) for x in (p.decay, p.beta1, p.beta2, p.min_weight, p.max_weight)])
        for d in (weights, m, v, grads):
            for k, a in d.items():
                assert a.dtype == self.real and a.flags.c_contiguous, k
        ws, _ = self._pack(desc, weights)
        ms, _ = self._pack(desc, m)
        vs, _ = self._pack(desc, v)
        gs, _ = self._pack(desc, grads)
        self.lib.orc_net_update(ctypes.byref(cdesc), ctypes.byref(ws), ctypes.byref(ms), ctypes.byref(vs),
                                ctypes.byref(gs), self._scalar(adj), self._scalar(rate), table)

    def train(self, desc, weights, batches, lr, hp, grad_factor=None):
        """Run AdamW steps over `batches` (iterable of (stm, nstm, buckets, targets)).

        Returns (weights, m, v, [loss_sum per step]); all state in this oracle's precision.
        """
        w = self.to_real(weights)
        m, v = self.zeros_like(desc), self.zeros_like(desc)
        losses = []
        for stm, nstm, buckets, targets in batches:
            loss, g, _ = self.net_grad(desc, w, stm, nstm, buckets, targets)
            adj = grad_factor if grad_factor is not None else 1.0 / len(targets)
            self.net_update(desc, w, m, v, g, adj, lr, hp)
            losses.append(loss)
        return w, m, v, losses
