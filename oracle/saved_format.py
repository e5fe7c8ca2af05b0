"""TEST INFRASTRUCTURE ONLY: numpy restatement of the reference's network export.

Follows jw1912/bullet crates/trainer/src/model/weights.rs:
  * QuantTarget::quantise           :281-331  (f64 product, round-half-away or truncate, must fit exactly)
  * SavedFormat::transpose_impl     :254-269
  * ModelWeights::to_quantised_buffer :158-177 (concatenate, pad to 64 bytes with "bullet")
and crates/bullet_lib/src/value/save.rs:45-69 (raw.bin: the named weights as f32, no transforms).
The reference has no test for these functions, so parity here is pinned by hand-computed cases
in tests/ ("parity unpinned" by reference vectors).
"""
import numpy as np

DTYPES = {"f32": np.dtype("<f4"), "i8": np.dtype("i1"), "i16": np.dtype("<i2"), "i32": np.dtype("<i4")}


class QuantisationError(ValueError):
    pass


def round_or_trunc(x: np.ndarray, rnd: bool) -> np.ndarray:
    t = np.trunc(x)
    if not rnd:
        return t
    # f64::round: half away from zero, decided on the exact fractional part
    return t + np.sign(x) * (np.abs(x - t) >= 0.5)


def quantise(values, target: str, multiplier: int, rnd: bool) -> bytes:
    v = np.asarray(values, dtype=np.float32).ravel()
    if target == "f32":
        return v.astype("<f4").tobytes()
    info = np.iinfo(DTYPES[target])
    with np.errstate(invalid="ignore"):
        qf = round_or_trunc(np.float64(multiplier) * v.astype(np.float64), rnd)
    ok = (qf >= info.min) & (qf <= info.max)  # NaN compares false
    if not ok.all():
        raise QuantisationError(f"Failed quantisation from f32 to {target}!")
    return qf.astype(DTYPES[target]).tobytes()


def transpose_impl(rows: int, cols: int, w) -> np.ndarray:
    w = np.asarray(w, dtype=np.float32).ravel()
    assert w.size == rows * cols
    out = np.zeros_like(w)
    for i in range(rows):
        out[cols * i:cols * i + cols] = w[i::rows][:cols]  # new[cols*i + j] = w[rows*j + i]
    return out


def entry_bytes(weights: dict, shapes: dict, fmt: dict) -> bytes:
    """fmt: {"custom": bytes} or {"id", "quant", "multiplier", "round", "transpose", "merge_factoriser"}."""
    if "custom" in fmt:
        return bytes(fmt["custom"])
    v = np.asarray(weights[fmt["id"]], dtype=np.float32).ravel()
    if fmt.get("merge_factoriser"):
        f = np.asarray(weights["l0f"], dtype=np.float32).ravel()
        v = (v + np.tile(f, v.size // f.size)).astype(np.float32)  # examples/progression/3_input_buckets.rs:46-53
    if fmt.get("transpose"):
        v = transpose_impl(*shapes[fmt["id"]], v)
    return quantise(v, fmt.get("quant", "f32"), fmt.get("multiplier", 1), bool(fmt.get("round")))


def to_quantised_buffer(weights: dict, shapes: dict, formats, pad: bool) -> bytes:
    buf = b"".join(entry_bytes(weights, shapes, f) for f in formats)
    if pad and len(buf) % 64:
        chs = b"bullet"
        buf += bytes(chs[i % 6] for i in range(64 - len(buf) % 64))
    return buf


def unquantised_buffer(weights: dict, formats) -> bytes:
    return b"".join(np.asarray(weights[f["id"]], dtype="<f4").tobytes() for f in formats if "id" in f)
