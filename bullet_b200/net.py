"""Python host side of the C ABI: `Net` wraps one `b200_net`, `featurise` wraps the mappers.

Method names follow the reference's trainer vocabulary: weights are addressed by their ids
("l0w", "l1b", ...), `set_params_for_weight` mirrors Optimiser::set_params_for_weight
(crates/trainer/src/optimiser.rs:204-206), `step` is one pass of the loop in
crates/trainer/src/run.rs:166-250.
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import _lib
from .configs import KING_BUCKETS_16, AdamWParams, CNetDesc, NetDesc

KIND_WEIGHT, KIND_MOMENTUM, KIND_VELOCITY, KIND_GRAD = 0, 1, 2, 3
FT_AUTO, FT_GATHER, FT_TILED = 0, 1, 2


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


class Net:
    def __init__(self, desc: NetDesc, device: int = 0, stream: int | None = None):
        self.lib = _lib.load()
        self.desc = desc
        self._h = ctypes.c_void_p()
        cdesc = CNetDesc.from_desc(desc)
        _lib.check(self.lib.b200_net_create(device, ctypes.c_void_p(stream or 0), ctypes.byref(cdesc),
                                            ctypes.byref(self._h)))

    def close(self) -> None:
        if self._h:
            self.lib.b200_net_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ----------------------------------------------------------------- tensors
    def set_option(self, key: str, value: int) -> None:
        _lib.check(self.lib.b200_net_set_option(self._h, key.encode(), value))

    def tensor_size(self, name: str) -> int:
        n = ctypes.c_int64()
        _lib.check(self.lib.b200_net_tensor_size(self._h, name.encode(), ctypes.byref(n)))
        return n.value

    def set_tensor(self, name: str, values, kind: int = KIND_WEIGHT) -> None:
        a = np.ascontiguousarray(values, dtype=np.float32).ravel()
        _lib.check(self.lib.b200_net_set_tensor(self._h, name.encode(), kind, _p(a), a.size))

    def get_tensor(self, name: str, kind: int = KIND_WEIGHT) -> np.ndarray:
        out = np.empty(self.tensor_size(name), dtype=np.float32)
        _lib.check(self.lib.b200_net_get_tensor(self._h, name.encode(), kind, _p(out), out.size))
        return out

    def load_weights(self, tensors: dict) -> None:
        for name in self.desc.tensor_shapes():
            self.set_tensor(name, tensors[name])

    def tensors(self, kind: int = KIND_WEIGHT) -> dict:
        return {name: self.get_tensor(name, kind) for name in self.desc.tensor_shapes()}

    def set_params_for_weight(self, name: str | None, p: AdamWParams) -> None:
        c = _lib.CAdamW(p.decay, p.beta1, p.beta2, p.min_weight, p.max_weight)
        _lib.check(self.lib.b200_net_set_adamw(self._h, name.encode() if name else None, ctypes.byref(c)))

    def set_optimiser_for_weight(self, name: str | None, params) -> None:
        """AdamWParams, RAdamParams or RangerParams for one weight (None: all), as the reference's
        `Optimiser::set_params_for_weight` does for whichever optimiser the trainer was built with."""
        from .configs import RAdamParams, RangerParams

        big = float(np.finfo(np.float32).max)
        if isinstance(params, RAdamParams):
            lo, hi = params.clip if params.clip is not None else (-big, big)
            c = _lib.COptimiser(1, params.decay, params.beta1, params.beta2, lo, hi, params.n_sma_threshold, 0.5, 6)
        elif isinstance(params, RangerParams):
            c = _lib.COptimiser(2, params.decay, params.beta1, params.beta2, params.min_weight, params.max_weight, 5.0,
                                params.alpha, params.k)
        else:
            c = _lib.COptimiser(0, params.decay, params.beta1, params.beta2, params.min_weight, params.max_weight, 5.0, 0.5, 6)
        _lib.check(self.lib.b200_net_set_optimiser(self._h, name.encode() if name else None, ctypes.byref(c)))

    # ------------------------------------------------------------------- batch
    def upload(self, slot: int, stm, nstm, buckets, targets) -> None:
        stm = np.ascontiguousarray(stm, dtype=np.int32)
        nstm = np.ascontiguousarray(nstm, dtype=np.int32)
        targets = np.ascontiguousarray(targets, dtype=np.float32)
        n = targets.size
        if stm.size != n * self.desc.nnz or nstm.size != n * self.desc.nnz:
            raise ValueError("index arrays must hold n * nnz slots")
        b = None if buckets is None else np.ascontiguousarray(buckets, dtype=np.int32)
        _lib.check(self.lib.b200_batch_upload(self._h, slot, _p(stm), _p(nstm), None if b is None else _p(b),
                                              _p(targets), n))

    # -------------------------------------------------------------------- step
    def upload_records(self, slot: int, game: str, records: np.ndarray, scale: float = 400.0, blend: float = 0.5,
                       on_device: bool = False) -> None:
        """Raw 32-byte records -> featurised, packed batch in the slot: one pass on all host cores, or
        (`on_device`) 32 bytes per position copied and everything else done by kernels on the copy stream."""
        records = np.ascontiguousarray(records)
        code = {"chess768": 0, "chess_buckets": 1, "ataxx147": 2}[game]
        layout = np.asarray(KING_BUCKETS_16, dtype=np.int32) if code == 1 else None
        fn = self.lib.b200_batch_upload_records_gpu if on_device else self.lib.b200_batch_upload_records
        _lib.check(fn(self._h, slot, _p(records), len(records), code, _p(layout) if layout is not None else None, scale, blend))

    def slot_contents(self, slot: int) -> dict:
        """Debug/inspection: what the slot holds on the device (packed lists, buckets, targets, the two orders)."""
        count = ctypes.c_int32()
        _lib.check(self.lib.b200_slot_read(self._h, slot, None, None, None, None, None, None, ctypes.byref(count)))
        n, nnz = count.value, self.desc.nnz
        out = {"stm": np.empty((n, nnz), np.uint16), "nstm": np.empty((n, nnz), np.uint16), "buckets": np.empty(n, np.int32),
               "targets": np.empty(n, np.float32), "order": np.empty(n, np.int32), "pair_order": np.empty(2 * n, np.int32)}
        _lib.check(self.lib.b200_slot_read(self._h, slot, _p(out["stm"]), _p(out["nstm"]), _p(out["buckets"]), _p(out["targets"]),
                                           _p(out["order"]), _p(out["pair_order"]), None))
        return out

    def step(self, slot: int, lr: float, grad_factor: float) -> None:
        _lib.check(self.lib.b200_step(self._h, slot, lr, grad_factor))

    def backward(self, slot: int) -> None:
        _lib.check(self.lib.b200_backward(self._h, slot))

    def update(self, lr: float, grad_factor: float) -> None:
        _lib.check(self.lib.b200_update(self._h, lr, grad_factor))

    # the same step in phases (see include/bullet_b200.h); used by the data-parallel host
    def forward_begin(self, slot: int) -> None:
        _lib.check(self.lib.b200_forward_begin(self._h, slot))

    def forward_ft(self, slot: int, part: int, n_parts: int) -> None:
        _lib.check(self.lib.b200_forward_ft(self._h, slot, part, n_parts))

    def tensor_range(self, name: str) -> tuple[int, int]:
        """(first float, count) of a tensor inside the flat buffers."""
        first, count = ctypes.c_int64(), ctypes.c_int64()
        _lib.check(self.lib.b200_net_tensor_offset(self._h, name.encode(), ctypes.byref(first)))
        _lib.check(self.lib.b200_net_tensor_size(self._h, name.encode(), ctypes.byref(count)))
        return first.value, count.value

    # the data-parallel update over peer memory (see include/bullet_b200.h)
    def exchange_export(self) -> bytes:
        buf = ctypes.create_string_buffer(192)
        _lib.check(self.lib.b200_exchange_export(self._h, buf, 192))
        return buf.raw

    def exchange_import(self, rank: int, world: int, handles: bytes) -> None:
        _lib.check(self.lib.b200_exchange_import(self._h, rank, world, handles, len(handles)))

    def update_exchange(self, lr: float, grad_factor: float) -> None:
        _lib.check(self.lib.b200_update_exchange(self._h, lr, grad_factor))

    def step_exchange(self, slot: int, lr: float, grad_factor: float) -> None:
        """One data-parallel step with the exchange hidden under the backward pass."""
        _lib.check(self.lib.b200_step_exchange(self._h, slot, lr, grad_factor))

    def update_exchange_range(self, lr: float, grad_factor: float, first: int, count: int, gather: bool, stream: int = 0) -> None:
        _lib.check(self.lib.b200_update_exchange_range(self._h, lr, grad_factor, first, count, int(gather),
                                                       ctypes.c_void_p(stream or 0)))

    def grad_zero_range(self, first: int, count: int) -> None:
        _lib.check(self.lib.b200_grad_zero_range(self._h, first, count))

    def backward_begin(self, slot: int) -> None:
        _lib.check(self.lib.b200_backward_begin(self._h, slot))

    def backward_ft(self, slot: int, part: int, n_parts: int) -> None:
        _lib.check(self.lib.b200_backward_ft(self._h, slot, part, n_parts))

    def backward_end(self, slot: int) -> None:
        _lib.check(self.lib.b200_backward_end(self._h, slot))

    def grad_part(self, part: int, n_parts: int) -> tuple[int, int]:
        first, count = ctypes.c_int64(), ctypes.c_int64()
        _lib.check(self.lib.b200_grad_part(self._h, part, n_parts, ctypes.byref(first), ctypes.byref(count)))
        return first.value, count.value

    def update_range(self, lr: float, grad_factor: float, first: int, count: int) -> None:
        _lib.check(self.lib.b200_update_range(self._h, lr, grad_factor, first, count))

    def update_end(self) -> None:
        _lib.check(self.lib.b200_update_end(self._h))

    def loss(self, steps_back: int = 0) -> float:
        """Summed loss of the most recent update (or of the one `steps_back` before it); waits for it."""
        v = ctypes.c_float()
        _lib.check(self.lib.b200_loss_of(self._h, steps_back, ctypes.byref(v)))
        return v.value

    def forward(self, slot: int, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.float32)
        _lib.check(self.lib.b200_forward(self._h, slot, _p(out)))
        return out

    def save_checkpoint(self, directory: str) -> None:
        """weights.bin / momentum.bin / velocity.bin in the reference's record format."""
        _lib.check(self.lib.b200_checkpoint_save(self._h, directory.encode()))

    def load_checkpoint(self, directory: str) -> None:
        _lib.check(self.lib.b200_checkpoint_load(self._h, directory.encode()))

    def tensor_shape(self, name: str):
        """(rows, cols) of a weight, column-major as the reference's Shape."""
        r, c = ctypes.c_int64(), ctypes.c_int64()
        _lib.check(self.lib.b200_net_tensor_shape(self._h, name.encode(), ctypes.byref(r), ctypes.byref(c)))
        return r.value, c.value

    def to_quantised_buffer(self, formats, pad: bool = True) -> bytes:
        """ModelWeights::to_quantised_buffer (crates/trainer/src/model/weights.rs:158-177)."""
        from .saved_format import c_formats

        arr, keep = c_formats(formats)
        size = ctypes.c_int64()
        _lib.check(self.lib.b200_saved_format_size(self._h, arr, len(formats), int(pad), ctypes.byref(size)))
        out = ctypes.create_string_buffer(max(1, size.value))
        _lib.check(self.lib.b200_saved_format_write(self._h, arr, len(formats), int(pad), out, size.value))
        del keep
        return out.raw[:size.value]

    def save_quantised(self, path: str, formats) -> None:
        from .saved_format import c_formats

        arr, keep = c_formats(formats)
        _lib.check(self.lib.b200_save_quantised(self._h, arr, len(formats), path.encode()))
        del keep

    def save_unquantised(self, path: str, formats) -> None:
        from .saved_format import c_formats

        arr, keep = c_formats(formats)
        _lib.check(self.lib.b200_save_unquantised(self._h, arr, len(formats), path.encode()))
        del keep

    def save_to_checkpoint(self, path: str, formats) -> None:
        """`path`/optimiser_state/{weights,momentum,velocity}.bin, raw.bin and quantised.bin
        (crates/bullet_lib/src/value/save.rs:24-43)."""
        import os

        os.makedirs(os.path.join(path, "optimiser_state"), exist_ok=True)
        self.save_checkpoint(os.path.join(path, "optimiser_state"))
        self.save_unquantised(os.path.join(path, "raw.bin"), formats)
        self.save_quantised(os.path.join(path, "quantised.bin"), formats)

    def sync(self) -> None:
        _lib.check(self.lib.b200_sync(self._h))

    def timings(self) -> dict:
        t = _lib.CTimings()
        _lib.check(self.lib.b200_get_timings(self._h, ctypes.byref(t)))
        return {name: getattr(t, name) for name, _ in t._fields_}

    def stat(self, key: str) -> int:
        v = ctypes.c_int64()
        _lib.check(self.lib.b200_net_get_stat(self._h, key.encode(), ctypes.byref(v)))
        return v.value

    def activation(self, which: int, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.float32)
        _lib.check(self.lib.b200_net_get_activation(self._h, which, _p(out), out.size))
        return out

    def flat_buffer(self, kind: int):
        """(device address, number of floats) of a flat buffer: weights, momentum, velocity or gradients."""
        ptr, n = ctypes.c_void_p(), ctypes.c_int64()
        _lib.check(self.lib.b200_flat_buffer(self._h, kind, ctypes.byref(ptr), ctypes.byref(n)))
        return ptr.value, n.value

    def grad_buffer(self):
        """(device address, number of floats) of the flat gradient buffer; the first float is the loss."""
        ptr, n = ctypes.c_void_p(), ctypes.c_int64()
        _lib.check(self.lib.b200_grad_buffer(self._h, ctypes.byref(ptr), ctypes.byref(n)))
        return ptr.value, n.value


def featurise(game: str, records: np.ndarray, desc: NetDesc, scale: float = 400.0, blend: float = 0.5):
    """records -> (stm, nstm, buckets, targets) in the reference mapper's layout."""
    lib = _lib.load()
    n = len(records)
    records = np.ascontiguousarray(records)
    stm = np.empty((n, desc.nnz), dtype=np.int32)
    nstm = np.empty((n, desc.nnz), dtype=np.int32)
    if game == "chess768":
        _lib.check(lib.b200_map_chess768(_p(records), n, _p(stm), _p(nstm), desc.nnz))
    elif game == "chess_buckets":
        layout = np.asarray(KING_BUCKETS_16, dtype=np.int32)
        _lib.check(lib.b200_map_chess_buckets_mirrored(_p(records), n, _p(layout), _p(stm), _p(nstm), desc.nnz))
    elif game == "ataxx147":
        _lib.check(lib.b200_map_ataxx147(_p(records), n, _p(stm), _p(nstm), desc.nnz))
    else:
        raise ValueError(game)
    buckets = np.zeros(n, dtype=np.int32)
    if desc.n_out_buckets > 1:
        _lib.check(lib.b200_material_count(_p(records), n, desc.n_out_buckets, _p(buckets)))
    targets = np.empty(n, dtype=np.float32)
    _lib.check(lib.b200_make_targets(_p(records), n, scale, blend, _p(targets)))
    return stm, nstm, buckets, targets


def probe_bandwidth(kind: str, nbytes: int, reps: int = 20, device: int = 0) -> float:
    """GB/s of repeated 16-byte loads ("read") or of reductions with 16, 4 or 8 bytes per lane ("atomic",
    "atomic4", "atomic8") over a buffer of `nbytes`."""
    out = ctypes.c_double()
    code = {"read": 0, "atomic": 1, "atomic4": 2, "atomic8": 3}[kind]
    _lib.check(_lib.load().b200_probe_bandwidth(device, code, nbytes, reps, ctypes.byref(out)))
    return out.value


def pack_indices(idx: np.ndarray) -> np.ndarray:
    idx = np.ascontiguousarray(idx, dtype=np.int32)
    out = np.empty(idx.shape, dtype=np.uint16)
    _lib.check(_lib.load().b200_pack_indices_u16(_p(idx), idx.size, _p(out)))
    return out


def unpack_indices(packed: np.ndarray) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint16)
    out = np.empty(packed.shape, dtype=np.int32)
    _lib.check(_lib.load().b200_unpack_indices_u16(_p(packed), packed.size, _p(out)))
    return out
