// Network export in the reference's `SavedFormat` scheme: the bytes an engine loads.
//
// Reference (jw1912/bullet): `SavedFormat` and `QuantTarget::quantise`
// (crates/trainer/src/model/weights.rs:183-335), `ModelWeights::to_quantised_buffer`
// (weights.rs:158-177: formats concatenated, then padded to a multiple of 64 bytes with the
// letters of "bullet"), `save_quantised` / `save_unquantised`
// (crates/bullet_lib/src/value/save.rs:45-88).  A format entry is either custom bytes or a
// weight id with transforms followed by quantisation:
//     value -> [merge the factoriser] -> [transpose] -> q = round_or_trunc(f64(mult) * f64(value))
//     -> stored as i8 / i16 / i32 little-endian; an entry that does not fit its type fails the
//     whole export ("Failed quantisation from f32 to i16!"), nothing is clamped.
// `round` is round-half-away-from-zero (Rust f64::round), otherwise truncation toward zero.
// Closures cannot cross a C ABI, so the two transforms every example uses are flags here: the
// factoriser merge of examples/progression/3_input_buckets.rs:46-53 and `transpose`
// (weights.rs:254-269).  Free-form transforms live in the C++ header, built on b200_quantise.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <limits>
#include <string>
#include <vector>

#include "../../include/bullet_b200.h"
#include "common.h"

namespace {

template <typename T>
int quantise_as(const float* v, int64_t n, int32_t mult, bool round, void* out, const char* type_name) {
    T* dst = static_cast<T*>(out);
    const double q = (double)mult;
    const double lo = (double)std::numeric_limits<T>::min(), hi = (double)std::numeric_limits<T>::max();
    for (int64_t i = 0; i < n; i++) {
        const double x = q * (double)v[i];
        const double qf = round ? std::round(x) : std::trunc(x);
        if (!(qf >= lo && qf <= hi))  // also catches NaN
            return b200::fail(B200_ERR_DATA, "Failed quantisation from f32 to %s! (element %lld: %g x %d)", type_name, (long long)i,
                              (double)v[i], (int)mult);
        dst[i] = (T)qf;
    }
    return 0;
}

int check_quant(int32_t quant, int32_t mult, const char* who) {
    if (quant < B200_QUANT_FLOAT || quant > B200_QUANT_I32) return b200::fail(B200_ERR_ARG, "%s: unknown quantisation target %d", who, quant);
    // the reference's multiplier is an i16 for i8 and i16 targets (weights.rs:343-358)
    if ((quant == B200_QUANT_I8 || quant == B200_QUANT_I16) && (mult < -32768 || mult > 32767))
        return b200::fail(B200_ERR_ARG, "%s: multiplier %d does not fit the 16 bits the i8 / i16 targets take", who, mult);
    return 0;
}

// transforms of one entry, in the order the examples apply them; `out` receives the floats to quantise
int entry_values(b200_net* net, const b200_saved_format& f, std::vector<float>& out) {
    int64_t n = 0, rows = 0, cols = 0;
    if (int rc = b200_net_tensor_size(net, f.id, &n)) return rc;
    if (int rc = b200_net_tensor_shape(net, f.id, &rows, &cols)) return rc;
    out.resize((size_t)n);
    if (int rc = b200_net_get_tensor(net, f.id, B200_KIND_WEIGHT, out.data(), n)) return rc;
    if (f.merge_factoriser) {
        int64_t nf = 0;
        if (b200_net_tensor_size(net, "l0f", &nf) != 0 || nf == 0 || n % nf != 0)
            return b200::fail(B200_ERR_ARG, "saved format: '%s' cannot take the factoriser (no l0f, or sizes do not divide)", f.id);
        std::vector<float> fac((size_t)nf);
        if (int rc = b200_net_get_tensor(net, "l0f", B200_KIND_WEIGHT, fac.data(), nf)) return rc;
        for (int64_t i = 0; i < n; i++) out[(size_t)i] = out[(size_t)i] + fac[(size_t)(i % nf)];  // a + b in fp32, as the example's zip
    }
    if (f.transpose) {
        std::vector<float> t((size_t)n);
        if (int rc = b200_transpose(out.data(), rows, cols, t.data())) return rc;
        out.swap(t);
    }
    return 0;
}

int write_file(const char* path, const std::vector<unsigned char>& bytes, const char* who) {
    FILE* f = std::fopen(path, "wb");
    if (!f) return b200::fail(B200_ERR_ARG, "%s: cannot create %s", who, path);
    const bool ok = bytes.empty() || std::fwrite(bytes.data(), 1, bytes.size(), f) == bytes.size();
    if (std::fclose(f) != 0 || !ok) return b200::fail(B200_ERR_ARG, "%s: short write to %s", who, path);
    return 0;
}

int build_buffer(b200_net* net, const b200_saved_format* fmt, int32_t n_fmt, int32_t pad, std::vector<unsigned char>& buf) {
    if (!net || (!fmt && n_fmt > 0) || n_fmt < 0) return b200::fail(B200_ERR_ARG, "saved format: null argument");
    buf.clear();
    std::vector<float> values;
    for (int32_t k = 0; k < n_fmt; k++) {
        const b200_saved_format& f = fmt[k];
        if (!f.id) {  // custom bytes: a header, padding, ...
            if (f.custom_len < 0 || (f.custom_len > 0 && !f.custom)) return b200::fail(B200_ERR_ARG, "saved format %d: custom bytes missing", k);
            const unsigned char* c = static_cast<const unsigned char*>(f.custom);
            buf.insert(buf.end(), c, c + f.custom_len);
            continue;
        }
        if (int rc = check_quant(f.quant, f.multiplier, "saved format")) return rc;
        if (int rc = entry_values(net, f, values)) return rc;
        const size_t at = buf.size();
        buf.resize(at + values.size() * (size_t)b200_quant_size(f.quant));
        if (int rc = b200_quantise(values.data(), (int64_t)values.size(), f.quant, f.multiplier, f.round, buf.data() + at)) return rc;
    }
    if (pad && buf.size() % 64) {  // weights.rs:165-174
        static const char chs[6] = {'b', 'u', 'l', 'l', 'e', 't'};
        const size_t extra = 64 - buf.size() % 64;
        for (size_t i = 0; i < extra; i++) buf.push_back((unsigned char)chs[i % 6]);
    }
    return 0;
}

}  // namespace

extern "C" {

int64_t b200_quant_size(int32_t quant) {
    switch (quant) {
        case B200_QUANT_FLOAT: return 4;
        case B200_QUANT_I8: return 1;
        case B200_QUANT_I16: return 2;
        case B200_QUANT_I32: return 4;
        default: return 0;
    }
}

int b200_quantise(const float* values, int64_t n, int32_t quant, int32_t multiplier, int32_t round, void* out) {
    if (n < 0 || (n > 0 && (!values || !out))) return b200::fail(B200_ERR_ARG, "quantise: null argument");
    if (int rc = check_quant(quant, multiplier, "quantise")) return rc;
    switch (quant) {
        case B200_QUANT_FLOAT: std::memcpy(out, values, (size_t)n * 4); return 0;  // little-endian host, as the format
        case B200_QUANT_I8: return quantise_as<int8_t>(values, n, multiplier, round != 0, out, "i8");
        case B200_QUANT_I16: return quantise_as<int16_t>(values, n, multiplier, round != 0, out, "i16");
        default: return quantise_as<int32_t>(values, n, multiplier, round != 0, out, "i32");
    }
}

int b200_transpose(const float* in, int64_t rows, int64_t cols, float* out) {
    if (rows < 0 || cols < 0 || ((rows * cols) > 0 && (!in || !out))) return b200::fail(B200_ERR_ARG, "transpose: bad argument");
    for (int64_t i = 0; i < rows; i++)
        for (int64_t j = 0; j < cols; j++) out[cols * i + j] = in[rows * j + i];
    return 0;
}

int b200_saved_format_size(b200_net* net, const b200_saved_format* fmt, int32_t n_fmt, int32_t pad, int64_t* bytes) {
    if (!net || !bytes || (!fmt && n_fmt > 0) || n_fmt < 0) return b200::fail(B200_ERR_ARG, "saved_format_size: null argument");
    int64_t total = 0;
    for (int32_t k = 0; k < n_fmt; k++) {
        if (!fmt[k].id) {
            if (fmt[k].custom_len < 0) return b200::fail(B200_ERR_ARG, "saved format %d: negative length", k);
            total += fmt[k].custom_len;
            continue;
        }
        if (int rc = check_quant(fmt[k].quant, fmt[k].multiplier, "saved format")) return rc;
        int64_t n = 0;
        if (int rc = b200_net_tensor_size(net, fmt[k].id, &n)) return rc;
        total += n * b200_quant_size(fmt[k].quant);
    }
    if (pad && total % 64) total += 64 - total % 64;
    *bytes = total;
    return 0;
}

int b200_saved_format_write(b200_net* net, const b200_saved_format* fmt, int32_t n_fmt, int32_t pad, void* out, int64_t out_bytes) {
    std::vector<unsigned char> buf;
    if (int rc = build_buffer(net, fmt, n_fmt, pad, buf)) return rc;
    if (!out || out_bytes < (int64_t)buf.size())
        return b200::fail(B200_ERR_ARG, "saved_format_write: the buffer holds %lld bytes, %lld are needed", (long long)out_bytes, (long long)buf.size());
    if (!buf.empty()) std::memcpy(out, buf.data(), buf.size());
    return 0;
}

int b200_save_quantised(b200_net* net, const b200_saved_format* fmt, int32_t n_fmt, const char* path) {
    if (!path) return b200::fail(B200_ERR_ARG, "save_quantised: null path");
    std::vector<unsigned char> buf;
    if (int rc = build_buffer(net, fmt, n_fmt, 1, buf)) return rc;
    return write_file(path, buf, "save_quantised");
}

int b200_save_unquantised(b200_net* net, const b200_saved_format* fmt, int32_t n_fmt, const char* path) {
    if (!net || !path || (!fmt && n_fmt > 0) || n_fmt < 0) return b200::fail(B200_ERR_ARG, "save_unquantised: null argument");
    std::vector<unsigned char> buf;
    std::vector<float> values;
    for (int32_t k = 0; k < n_fmt; k++) {
        if (!fmt[k].id) continue;  // only entries that name a weight; no transforms, no padding (save.rs:45-69)
        int64_t n = 0;
        if (int rc = b200_net_tensor_size(net, fmt[k].id, &n)) return rc;
        values.resize((size_t)n);
        if (int rc = b200_net_get_tensor(net, fmt[k].id, B200_KIND_WEIGHT, values.data(), n)) return rc;
        const unsigned char* c = reinterpret_cast<const unsigned char*>(values.data());
        buf.insert(buf.end(), c, c + (size_t)n * 4);
    }
    return write_file(path, buf, "save_unquantised");
}

}  // extern "C"
