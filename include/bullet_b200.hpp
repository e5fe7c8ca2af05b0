// C++ host layer over the C ABI (bullet_b200.h): the part of bullet's builder API that the
// value-net examples use, enough to write a network the way the reference's examples do, and
// a recogniser that turns the resulting graph into a b200_net_desc.
//
// Mirrored reference interface (jw1912/bullet): ModelBuilder::{new_affine, new_weights}
// (crates/compiler/src/model/builder.rs:95-119), Affine::{forward, slice} (builder.rs:128-153),
// ModelNode::{crelu, screlu, sigmoid, concat, select, slice_rows, repeat, pairwise_mul,
// squared_error, +, *} (builder.rs:155-425), AdamWParams (crates/trainer/src/optimiser/adam.rs:20-33),
// Optimiser::set_params_for_weight (crates/trainer/src/optimiser.rs:204-206).
// Where the reference compiles any graph, this layer recognises ONE family — shared sparse
// affine on both perspectives, CReLU/SCReLU or pairwise CReLU, concat, one to three
// output-bucketed dense layers, sigmoid squared error — and refuses everything else with an
// error that says what it did not recognise; nothing is ever silently trained differently.
#pragma once
#include <cstdint>
#include <cstdio>
#include <functional>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <vector>

#include "bullet_b200.h"

namespace bullet {

struct Shape {
    int rows = 0, cols = 1;
    Shape() = default;
    Shape(int r, int c) : rows(r), cols(c) {}
};

enum class InitSettings { Zeroed, Normal };

struct AdamWParams {  // adam.rs:20-33
    float decay = 0.01f, beta1 = 0.9f, beta2 = 0.999f, min_weight = -1.98f, max_weight = 1.98f;
};

class GraphError : public std::runtime_error {
    using std::runtime_error::runtime_error;
};

namespace detail {
enum class Op { SparseInput, DenseInput, Weight, Matmul, Add, Mul, Slice, Repeat, CReLU, SCReLU, Sigmoid, Concat, Select, Sub };
struct Expr {
    Op op;
    int rows = 0, cols = 1;
    std::string id;  // inputs and weights
    int a = 0, b = 0;  // slice bounds / repeat count / nnz of a sparse input
    std::shared_ptr<Expr> lhs, rhs;
};
using E = std::shared_ptr<Expr>;
inline E make(Op op, int rows, int cols, E l = nullptr, E r = nullptr) {
    auto e = std::make_shared<Expr>();
    e->op = op, e->rows = rows, e->cols = cols, e->lhs = std::move(l), e->rhs = std::move(r);
    return e;
}
}  // namespace detail

class ModelNode {
   public:
    ModelNode() = default;
    explicit ModelNode(detail::E e) : e_(std::move(e)) {}
    const detail::E& expr() const { return e_; }
    int rows() const { return e_->rows; }

    ModelNode crelu() const { return unary(detail::Op::CReLU); }
    ModelNode screlu() const { return unary(detail::Op::SCReLU); }
    ModelNode sigmoid() const { return unary(detail::Op::Sigmoid); }
    ModelNode slice_rows(int start, int end) const {
        if (start < 0 || end > e_->rows || start >= end) throw GraphError("slice_rows: bounds outside the node");
        auto e = detail::make(detail::Op::Slice, end - start, e_->cols, e_);
        e->a = start, e->b = end;
        return ModelNode(e);
    }
    ModelNode repeat(int reps) const {  // builder.rs:421-424: tiles the columns
        auto e = detail::make(detail::Op::Repeat, e_->rows, e_->cols * reps, e_);
        e->a = reps;
        return ModelNode(e);
    }
    ModelNode pairwise_mul() const { return slice_rows(0, e_->rows / 2) * slice_rows(e_->rows / 2, e_->rows); }
    ModelNode concat(const ModelNode& rhs) const {
        if (e_->cols != 1 || rhs.e_->cols != 1) throw GraphError("concat: only column vectors");
        return ModelNode(detail::make(detail::Op::Concat, e_->rows + rhs.e_->rows, 1, e_, rhs.e_));
    }
    ModelNode select(const ModelNode& indices) const {  // builder.rs:395-414
        if (indices.e_->op != detail::Op::SparseInput || indices.e_->a != 1) throw GraphError("select: indices must be a sparse input with one slot");
        if (e_->rows % indices.e_->rows) throw GraphError("select: rows are not a multiple of the bucket count");
        return ModelNode(detail::make(detail::Op::Select, e_->rows / indices.e_->rows, 1, e_, indices.e_));
    }
    ModelNode squared_error(const ModelNode& target) const {  // builder.rs:351-354
        auto diff = detail::make(detail::Op::Sub, e_->rows, 1, e_, target.e_);
        return ModelNode(detail::make(detail::Op::Mul, e_->rows, 1, diff, diff));
    }
    ModelNode matmul(const ModelNode& x) const {
        if (e_->cols != x.e_->rows) throw GraphError("matmul: inner dimensions differ");
        return ModelNode(detail::make(detail::Op::Matmul, e_->rows, 1, e_, x.e_));
    }
    friend ModelNode operator+(const ModelNode& l, const ModelNode& r) {
        if (l.e_->rows != r.e_->rows || l.e_->cols != r.e_->cols) throw GraphError("+: shapes differ");
        return ModelNode(detail::make(detail::Op::Add, l.e_->rows, l.e_->cols, l.e_, r.e_));
    }
    friend ModelNode operator*(const ModelNode& l, const ModelNode& r) {
        if (l.e_->rows != r.e_->rows) throw GraphError("*: shapes differ");
        return ModelNode(detail::make(detail::Op::Mul, l.e_->rows, l.e_->cols, l.e_, r.e_));
    }

   private:
    ModelNode unary(detail::Op op) const { return ModelNode(detail::make(op, e_->rows, e_->cols, e_)); }
    detail::E e_;
};

struct Affine {  // builder.rs:128-153
    ModelNode weights, bias;
    Affine slice(int start, int end) const { return {weights.slice_rows(start, end), bias.slice_rows(start, end)}; }
    ModelNode forward(const ModelNode& input) const { return weights.matmul(input) + bias; }
};

class ModelBuilder {
   public:
    ModelNode new_weights(const std::string& id, Shape shape, InitSettings = InitSettings::Normal) {
        auto e = detail::make(detail::Op::Weight, shape.rows, shape.cols);
        e->id = id;
        return ModelNode(e);
    }
    Affine new_affine(const std::string& id, int input_size, int output_size) {  // builder.rs:104-119
        return {new_weights(id + "w", Shape(output_size, input_size)), new_weights(id + "b", Shape(output_size, 1), InitSettings::Zeroed)};
    }
    // ModelInputs::add_sparse / add_dense (crates/trainer/src/model/inputs.rs)
    ModelNode sparse_input(const std::string& id, int size, int nnz) {
        auto e = detail::make(detail::Op::SparseInput, size, 1);
        e->id = id, e->a = nnz;
        return ModelNode(e);
    }
    ModelNode dense_input(const std::string& id, int size) {
        auto e = detail::make(detail::Op::DenseInput, size, 1);
        e->id = id;
        return ModelNode(e);
    }
};

// ------------------------------------------------------------------ recogniser
namespace detail {
struct FtHalf {
    E table_w, table_f, bias, input;  // l0w, optional l0f (tiled), l0b, sparse input
    int act = 0;                      // B200_ACT_*
    bool pairwise = false;
    int H = 0;
};
inline bool same(const E& a, const E& b) { return a.get() == b.get(); }
inline const E& strip_slice(const E& e, int a, int b, const char* what) {
    if (e->op != Op::Slice || e->a != a || e->b != b) throw GraphError(std::string("pairwise: unexpected slice of ") + what);
    return e->lhs;
}
// W may be `l0w` or `l0w + l0f.repeat(n)`
inline void parse_table(const E& w, FtHalf& h) {
    if (w->op == Op::Weight) {
        h.table_w = w;
    } else if (w->op == Op::Add && w->lhs->op == Op::Weight && w->rhs->op == Op::Repeat && w->rhs->lhs->op == Op::Weight) {
        h.table_w = w->lhs;
        h.table_f = w->rhs->lhs;
        if (h.table_f->rows != h.table_w->rows || h.table_f->cols * w->rhs->a != h.table_w->cols)
            throw GraphError("factoriser: l0f.repeat(n) does not tile l0w");
    } else {
        throw GraphError("feature transformer: weights are neither a weight nor weight + weight.repeat(n)");
    }
}
// affine = W.matmul(sparse input) + b
inline void parse_affine(const E& e, E& w, E& b, E& x) {
    if (e->op != Op::Add || e->lhs->op != Op::Matmul) throw GraphError("expected `weights.matmul(x) + bias`");
    w = e->lhs->lhs, x = e->lhs->rhs, b = e->rhs;
}
inline int act_of(Op op) { return op == Op::CReLU ? B200_ACT_CRELU : op == Op::SCReLU ? B200_ACT_SCRELU : -1; }

inline FtHalf parse_ft(const E& e) {
    FtHalf h;
    E w, b, x;
    if (act_of(e->op) > 0) {  // act(l0.forward(input))
        parse_affine(e->lhs, w, b, x);
        h.act = act_of(e->op);
        parse_table(w, h);
        h.bias = b, h.input = x, h.H = w->rows;
    } else if (e->op == Op::Mul) {
        h.pairwise = true;
        h.act = B200_ACT_CRELU;
        const E &l = e->lhs, &r = e->rhs;
        if (l->op == Op::Slice && r->op == Op::Slice) {  // l0.forward(x).crelu().pairwise_mul()
            const E& u = l->lhs;
            if (!same(u, r->lhs) || u->op != Op::CReLU) throw GraphError("pairwise_mul must follow crelu()");
            h.H = u->rows;
            if (l->a != 0 || l->b != h.H / 2 || r->a != h.H / 2 || r->b != h.H) throw GraphError("pairwise_mul: halves expected");
            parse_affine(u->lhs, w, b, x);
            parse_table(w, h);
            h.bias = b, h.input = x;
        } else if (l->op == Op::CReLU && r->op == Op::CReLU) {  // l0.slice(0,h/2).forward(x).crelu() * l0.slice(h/2,h)...
            E w0, b0, x0, w1, b1, x1;
            parse_affine(l->lhs, w0, b0, x0);
            parse_affine(r->lhs, w1, b1, x1);
            if (!same(x0, x1)) throw GraphError("pairwise: the two halves read different inputs");
            if (w0->op != Op::Slice || w1->op != Op::Slice || b0->op != Op::Slice || b1->op != Op::Slice ||
                !same(w0->lhs, w1->lhs) || !same(b0->lhs, b1->lhs))
                throw GraphError("pairwise: the two halves must be slices of one affine layer");
            h.H = w0->lhs->rows;
            strip_slice(w0, 0, h.H / 2, "weights"), strip_slice(w1, h.H / 2, h.H, "weights");
            h.bias = strip_slice(b0, 0, h.H / 2, "bias");
            strip_slice(b1, h.H / 2, h.H, "bias");
            parse_table(w0->lhs, h);
            h.input = x0;
        } else {
            throw GraphError("a product of two nodes is only recognised as pairwise_mul of a crelu");
        }
        if (h.H % 2) throw GraphError("pairwise: odd hidden size");
    } else {
        throw GraphError("feature transformer: expected crelu/screlu of an affine layer, or their pairwise product");
    }
    if (h.input->op != Op::SparseInput) throw GraphError("feature transformer: input is not sparse");
    if (h.bias->op != Op::Weight) throw GraphError("feature transformer: bias is not a weight");
    return h;
}
}  // namespace detail

struct RecognisedNet {
    b200_net_desc desc{};
    std::vector<std::string> weight_ids;  // the graph's weight ids, in the order l0w, l0b, [l0f], l1w, l1b, ...
    // the name the C ABI knows each of them by (the reference's own ids when the graph uses them)
    std::vector<std::string> abi_names() const {
        std::vector<std::string> names = {"l0w", "l0b"};
        if (desc.factoriser_rows) names.push_back("l0f");
        for (int i = 1; i <= desc.n_dense; i++) {
            names.push_back("l" + std::to_string(i) + "w");
            names.push_back("l" + std::to_string(i) + "b");
        }
        return names;
    }
};

// `output` is what the builder closure returns (the raw network output); the loss is
// output.sigmoid().squared_error(targets), as ValueTrainerBuilder::loss_fn sets it in every
// example (examples/simple.rs:33).  `ft_block_rows` is a property of the input featuriser
// (768 for the chess input sets), not of the graph.
inline RecognisedNet recognise(const ModelNode& output, int ft_block_rows, int max_batch) {
    using namespace detail;
    RecognisedNet out;
    b200_net_desc& d = out.desc;
    struct Layer {
        E w, b;
        int act, rows_per_bucket;
    };
    std::vector<Layer> layers;
    E node = output.expr();
    int buckets = 1;
    E bucket_input;
    for (int guard = 0; guard < 8; guard++) {
        if (node->op == Op::Concat) break;
        Layer l{};
        l.act = B200_ACT_NONE;
        if (act_of(node->op) > 0) {
            l.act = act_of(node->op);
            node = node->lhs;
        }
        if (node->op == Op::Select) {
            if (bucket_input && !same(bucket_input, node->rhs)) throw GraphError("dense layers select by different inputs");
            bucket_input = node->rhs;
            buckets = bucket_input->rows;
            node = node->lhs;
        }
        E x;
        parse_affine(node, l.w, l.b, x);
        if (l.w->op != Op::Weight || l.b->op != Op::Weight) throw GraphError("dense layer: weights and bias must be plain weights");
        layers.push_back(l);
        node = x;
    }
    if (node->op != Op::Concat) throw GraphError("no stm|nstm concat found under the dense layers (skip connections are not recognised)");
    if (layers.empty() || layers.size() > 3) throw GraphError("one to three dense layers are supported");
    FtHalf s = parse_ft(node->lhs), n = parse_ft(node->rhs);
    if (!same(s.table_w, n.table_w) || !same(s.bias, n.bias) || s.act != n.act || s.pairwise != n.pairwise ||
        s.table_f.get() != n.table_f.get())
        throw GraphError("the two perspectives must share one feature transformer");
    if (same(s.input, n.input)) throw GraphError("both halves of the concat read the same input");
    if (s.input->rows != n.input->rows || s.input->a != n.input->a) throw GraphError("perspective inputs differ in size");
    d.n_inputs = s.input->rows;
    d.nnz = s.input->a;
    d.ft_out = s.H;
    d.ft_act = s.act;
    d.pairwise = s.pairwise;
    d.factoriser_rows = s.table_f ? s.table_f->cols : 0;
    d.n_out_buckets = buckets;
    d.n_dense = (int)layers.size();
    out.weight_ids = {s.table_w->id, s.bias->id};
    if (s.table_f) out.weight_ids.push_back(s.table_f->id);
    int in = s.pairwise ? s.H : 2 * s.H;
    for (int i = 0; i < d.n_dense; i++) {
        const Layer& l = layers[layers.size() - 1 - i];  // collected from the output downwards
        if (l.w->cols != in) throw GraphError("dense layer " + std::to_string(i + 1) + ": input size does not match the layer below");
        if (l.w->rows % buckets) throw GraphError("dense layer rows are not a multiple of the bucket count");
        d.dense_out[i] = l.w->rows / buckets;
        d.dense_act[i] = l.act;
        in = d.dense_out[i];
        out.weight_ids.push_back(l.w->id);
        out.weight_ids.push_back(l.b->id);
    }
    if (d.dense_out[d.n_dense - 1] != 1) throw GraphError("the network output must be one value per position");
    d.ft_block_rows = ft_block_rows;
    d.max_batch = max_batch;
    return out;
}

// ------------------------------------------------------------------ trainer handle
// ---- network export: crates/trainer/src/model/weights.rs:183-335 (SavedFormat, QuantTarget)
// A read-only view of the trained weights that transforms receive, as `&ModelWeights` in the reference.
struct WeightStore {
    struct Entry {
        std::vector<float> values;
        Shape shape;
    };
    std::map<std::string, Entry> stores;
    const Entry& get(const std::string& id) const {
        auto it = stores.find(id);
        if (it == stores.end()) throw std::runtime_error("no weight with id '" + id + "'");
        return it->second;
    }
};

class SavedFormat {
   public:
    using Transform = std::function<std::vector<float>(const WeightStore&, std::vector<float>)>;

    // custom bytes: a network header, padding, ...
    static SavedFormat custom(std::vector<uint8_t> bytes) {
        SavedFormat f;
        f.custom_ = std::move(bytes);
        f.is_custom_ = true;
        return f;
    }
    // starts from the values of weight `id`
    static SavedFormat id(const std::string& id) {
        SavedFormat f;
        f.id_ = id;
        f.has_id_ = true;
        return f.transform([id](const WeightStore& store, std::vector<float>) { return store.get(id).values; });
    }
    // starts from nothing: for formats that interleave several weights in a transform
    static SavedFormat empty() { return SavedFormat(); }

    // if quantising, round rather than truncate
    SavedFormat round() const {
        SavedFormat f(*this);
        f.no_custom();
        f.round_flag_ = true;
        return f;
    }
    template <typename T>
    SavedFormat quantise(int32_t multiplier) const {
        static_assert(std::is_same<T, int8_t>::value || std::is_same<T, int16_t>::value || std::is_same<T, int32_t>::value,
                      "quantise<int8_t | int16_t | int32_t>");
        SavedFormat f(*this);
        f.no_custom();
        f.quant_ = std::is_same<T, int8_t>::value ? B200_QUANT_I8 : std::is_same<T, int16_t>::value ? B200_QUANT_I16 : B200_QUANT_I32;
        f.multiplier_ = multiplier;
        return f;
    }
    // transposes the current values using the shape of this format's weight
    SavedFormat transpose() const {
        if (!has_id_) throw std::logic_error("SavedFormat::transpose needs a weight id");
        const std::string id = id_;
        return transform([id](const WeightStore& store, std::vector<float> w) {
            const Shape sh = store.get(id).shape;
            std::vector<float> out(w.size());
            if (b200_transpose(w.data(), (int64_t)sh.rows, (int64_t)sh.cols, out.data()) < 0) throw std::runtime_error(b200_last_error());
            return out;
        });
    }
    SavedFormat transform(Transform f) const {
        SavedFormat g(*this);
        g.no_custom();
        g.transforms_.push_back(std::move(f));
        return g;
    }
    bool has_id() const { return has_id_; }
    const std::string& get_id() const { return id_; }

    // SavedFormat::write_to_byte_buffer: transforms in order, then quantisation
    std::vector<uint8_t> write_to_byte_buffer(const WeightStore& store) const {
        if (is_custom_) return custom_;
        std::vector<float> w;
        for (const auto& t : transforms_) w = t(store, std::move(w));
        std::vector<uint8_t> out(w.size() * (size_t)b200_quant_size(quant_));
        if (b200_quantise(w.data(), (int64_t)w.size(), quant_, multiplier_, round_flag_ ? 1 : 0, out.data()) < 0)
            throw std::runtime_error(b200_last_error());
        return out;
    }

   private:
    void no_custom() const {
        if (is_custom_) throw std::logic_error("custom bytes take no transform or quantisation");
    }
    bool is_custom_ = false, has_id_ = false, round_flag_ = false;
    std::vector<uint8_t> custom_;
    std::string id_;
    int32_t quant_ = B200_QUANT_FLOAT, multiplier_ = 1;
    std::vector<Transform> transforms_;
};

// ModelWeights::to_quantised_buffer (weights.rs:158-177)
inline std::vector<uint8_t> to_quantised_buffer(const WeightStore& store, const std::vector<SavedFormat>& format, bool pad) {
    std::vector<uint8_t> buf;
    for (const auto& f : format) {
        const auto part = f.write_to_byte_buffer(store);
        buf.insert(buf.end(), part.begin(), part.end());
    }
    if (pad && buf.size() % 64) {
        static const char chs[6] = {'b', 'u', 'l', 'l', 'e', 't'};
        const size_t extra = 64 - buf.size() % 64;
        for (size_t i = 0; i < extra; i++) buf.push_back((uint8_t)chs[i % 6]);
    }
    return buf;
}

class Trainer {
   public:
    Trainer(const RecognisedNet& net, int device = 0) : ids_(net.weight_ids) {
        const auto names = net.abi_names();
        for (size_t i = 0; i < ids_.size(); i++) abi_[ids_[i]] = names[i];
        check(b200_net_create(device, nullptr, &net.desc, &h_));
    }
    ~Trainer() { b200_net_destroy(h_); }
    Trainer(const Trainer&) = delete;
    Trainer& operator=(const Trainer&) = delete;

    // weights are addressed by the ids the graph gave them, as in the reference
    void load_weights(const std::string& id, const std::vector<float>& v) {
        check(b200_net_set_tensor(h_, abi(id), B200_KIND_WEIGHT, v.data(), (int64_t)v.size()));
    }
    std::vector<float> weights(const std::string& id) {
        int64_t n = 0;
        check(b200_net_tensor_size(h_, abi(id), &n));
        std::vector<float> v((size_t)n);
        check(b200_net_get_tensor(h_, abi(id), B200_KIND_WEIGHT, v.data(), n));
        return v;
    }
    void set_params_for_weight(const std::string& id, const AdamWParams& p) {  // optimiser.rs:204-206
        const b200_adamw_params c{p.decay, p.beta1, p.beta2, p.min_weight, p.max_weight};
        check(b200_net_set_adamw(h_, abi(id), &c));
    }
    void upload(int slot, const int32_t* stm, const int32_t* nstm, const int32_t* buckets, const float* targets, int n) {
        check(b200_batch_upload(h_, slot, stm, nstm, buckets, targets, n));
    }
    // one pass of the loop in crates/trainer/src/run.rs:166-250; returns loss / batch as run.rs:221 logs it
    float step(int slot, int batch_size, float lr) {
        check(b200_step(h_, slot, lr, 1.0f / (float)batch_size));
        float loss = 0.f;
        check(b200_loss(h_, &loss));
        return loss / (float)batch_size;
    }
    std::vector<float> eval(int slot, int n) {
        std::vector<float> out((size_t)n);
        check(b200_forward(h_, slot, out.data()));
        return out;
    }
    // the trained weights on the host, under the ids of the graph (Optimiser::cpu_weights)
    WeightStore cpu_weights() {
        WeightStore store;
        for (const auto& id : ids_) {
            WeightStore::Entry e;
            e.values = weights(id);
            int64_t rows = 0, cols = 0;
            check(b200_net_tensor_shape(h_, abi(id), &rows, &cols));
            e.shape = Shape{(int)rows, (int)cols};
            store.stores[id] = std::move(e);
        }
        return store;
    }
    // crates/bullet_lib/src/value/save.rs:45-88
    void save_quantised(const std::string& path, const std::vector<SavedFormat>& format) {
        write_file(path, to_quantised_buffer(cpu_weights(), format, true));
    }
    void save_unquantised(const std::string& path, const std::vector<SavedFormat>& format) {
        std::vector<uint8_t> buf;
        for (const auto& f : format)
            if (f.has_id()) {
                const auto v = weights(f.get_id());
                const uint8_t* p = reinterpret_cast<const uint8_t*>(v.data());
                buf.insert(buf.end(), p, p + v.size() * sizeof(float));
            }
        write_file(path, buf);
    }
    const std::vector<std::string>& weight_ids() const { return ids_; }
    b200_net* handle() { return h_; }

   private:
    static void check(int rc) {
        if (rc < 0) throw std::runtime_error(std::string("bullet_b200 error ") + std::to_string(rc) + ": " + b200_last_error());
    }
    static void write_file(const std::string& path, const std::vector<uint8_t>& bytes) {
        FILE* f = std::fopen(path.c_str(), "wb");
        if (!f) throw std::runtime_error("cannot create " + path);
        const bool ok = bytes.empty() || std::fwrite(bytes.data(), 1, bytes.size(), f) == bytes.size();
        if (std::fclose(f) != 0 || !ok) throw std::runtime_error("short write to " + path);
    }
    const char* abi(const std::string& id) const {
        auto it = abi_.find(id);
        if (it == abi_.end()) throw std::runtime_error("no weight with id '" + id + "' in this network");
        return it->second.c_str();
    }
    b200_net* h_ = nullptr;
    std::vector<std::string> ids_;
    std::map<std::string, std::string> abi_;
};

}  // namespace bullet
