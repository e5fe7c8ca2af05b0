// Exercises the C++ host layer: networks written as the reference's examples write them are
// recognised into the expected b200_net_desc, and graphs outside the supported family are
// refused.  With the argument "gpu" it also trains one step on the device and prints the
// loss per position, which the Python test compares with the ctypes path.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <string>
#include <vector>

#include "bullet_b200.hpp"

using namespace bullet;

static int failures = 0;
#define EXPECT(cond)                                                        \
    do {                                                                    \
        if (!(cond)) {                                                      \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);   \
            failures++;                                                     \
        }                                                                   \
    } while (0)

static bool refused(const std::function<void()>& f, const char* needle) {
    try {
        f();
    } catch (const GraphError& e) {
        return std::strstr(e.what(), needle) != nullptr;
    }
    return false;
}

// examples/simple.rs:38-49
static ModelNode simple_net(ModelBuilder& b, ModelNode stm, ModelNode ntm, int hl) {
    Affine l0 = b.new_affine("l0", 768, hl), l1 = b.new_affine("l1", 2 * hl, 1);
    ModelNode stm_hidden = l0.forward(stm).screlu(), ntm_hidden = l0.forward(ntm).screlu();
    return l1.forward(stm_hidden.concat(ntm_hidden));
}

// examples/progression/4_multi_layer.rs:66-87; `fast` picks the sliced-affine spelling of pairwise
static ModelNode multi_layer_net(ModelBuilder& b, ModelNode stm, ModelNode ntm, ModelNode buckets, int hl, bool fast) {
    const int NB = 16, OB = 8, L2 = 16;
    ModelNode l0f = b.new_weights("l0f", Shape(hl, 768), InitSettings::Zeroed);
    Affine l0 = b.new_affine("l0", 768 * NB, hl);
    l0.weights = l0.weights + l0f.repeat(NB);
    Affine l1 = b.new_affine("l1", hl, OB * L2), l2 = b.new_affine("l2", L2, OB * 32), l3 = b.new_affine("l3", 32, OB);
    auto ft = [&](ModelNode in, int s, int e) { return l0.slice(s, e).forward(in).crelu(); };
    ModelNode sh = fast ? ft(stm, 0, hl / 2) * ft(stm, hl / 2, hl) : l0.forward(stm).crelu().pairwise_mul();
    ModelNode nh = fast ? ft(ntm, 0, hl / 2) * ft(ntm, hl / 2, hl) : l0.forward(ntm).crelu().pairwise_mul();
    ModelNode hl2 = l1.forward(sh.concat(nh)).select(buckets).screlu();
    ModelNode hl3 = l2.forward(hl2).select(buckets).screlu();
    return l3.forward(hl3).select(buckets);
}

int main(int argc, char** argv) {
    ModelBuilder b;
    {   // simple.rs
        ModelNode stm = b.sparse_input("stm", 768, 32), ntm = b.sparse_input("nstm", 768, 32);
        RecognisedNet r = recognise(simple_net(b, stm, ntm, 128), 768, 16384);
        EXPECT(r.desc.n_inputs == 768 && r.desc.nnz == 32 && r.desc.ft_out == 128 && r.desc.ft_act == B200_ACT_SCRELU);
        EXPECT(!r.desc.pairwise && r.desc.factoriser_rows == 0 && r.desc.n_out_buckets == 1 && r.desc.n_dense == 1);
        EXPECT(r.desc.dense_out[0] == 1 && r.desc.dense_act[0] == B200_ACT_NONE);
        EXPECT(r.weight_ids == (std::vector<std::string>{"l0w", "l0b", "l1w", "l1b"}));
    }
    {   // ataxx.rs shape (147 inputs, 49 slots)
        ModelNode stm = b.sparse_input("stm", 147, 49), ntm = b.sparse_input("ntm", 147, 49);
        Affine l0 = b.new_affine("l0", 147, 256), l1 = b.new_affine("l1", 512, 1);
        RecognisedNet r = recognise(l1.forward(l0.forward(stm).crelu().concat(l0.forward(ntm).crelu())), 147, 32768);
        EXPECT(r.desc.n_inputs == 147 && r.desc.nnz == 49 && r.desc.ft_out == 256 && r.desc.ft_act == B200_ACT_CRELU);
    }
    for (int fast = 0; fast < 2; fast++) {  // both spellings of pairwise give the same description
        ModelNode stm = b.sparse_input("stm", 12288, 32), ntm = b.sparse_input("nstm", 12288, 32);
        ModelNode buckets = b.sparse_input("buckets", 8, 1);
        RecognisedNet r = recognise(multi_layer_net(b, stm, ntm, buckets, 2048, fast), 768, 16384);
        EXPECT(r.desc.n_inputs == 12288 && r.desc.ft_out == 2048 && r.desc.pairwise == 1 && r.desc.ft_act == B200_ACT_CRELU);
        EXPECT(r.desc.factoriser_rows == 768 && r.desc.n_out_buckets == 8 && r.desc.n_dense == 3);
        EXPECT(r.desc.dense_out[0] == 16 && r.desc.dense_out[1] == 32 && r.desc.dense_out[2] == 1);
        EXPECT(r.desc.dense_act[0] == B200_ACT_SCRELU && r.desc.dense_act[1] == B200_ACT_SCRELU && r.desc.dense_act[2] == B200_ACT_NONE);
        EXPECT(r.weight_ids == (std::vector<std::string>{"l0w", "l0b", "l0f", "l1w", "l1b", "l2w", "l2b", "l3w", "l3b"}));
    }
    {   // refused: a skip connection around the dense layer (the shape of examples/tests/test2.rs:50-65)
        ModelNode stm = b.sparse_input("stm", 768, 32), ntm = b.sparse_input("nstm", 768, 32);
        Affine l0 = b.new_affine("l0", 768, 64), l1 = b.new_affine("l1", 128, 1);
        ModelNode hidden = l0.forward(stm).screlu().concat(l0.forward(ntm).screlu());
        ModelNode out = l1.forward(hidden) + l1.forward(hidden * hidden);
        EXPECT(refused([&] { recognise(out, 768, 1024); }, "expected"));
        // refused: different feature transformers per perspective
        Affine other = b.new_affine("lx", 768, 64);
        EXPECT(refused([&] { recognise(l1.forward(l0.forward(stm).screlu().concat(other.forward(ntm).screlu())), 768, 1024); },
                       "share one feature transformer"));
        // refused: an activation the kernels do not implement on the transformer output
        EXPECT(refused([&] { recognise(l1.forward(l0.forward(stm).sigmoid().concat(l0.forward(ntm).sigmoid())), 768, 1024); },
                       "feature transformer"));
        // refused: both halves read the same perspective
        EXPECT(refused([&] { recognise(l1.forward(l0.forward(stm).screlu().concat(l0.forward(stm).screlu())), 768, 1024); },
                       "same input"));
        EXPECT(refused([&] { l0.weights.matmul(b.sparse_input("bad", 5, 1)); }, "inner dimensions"));
    }
    {   // SavedFormat on a hand-made store: transforms in order, quantisation last (weights.rs:183-335)
        WeightStore store;
        store.stores["w"] = {{0.5f, -0.5f, 0.25f, 1.0f, -1.0f, 0.1f}, Shape(2, 3)};  // column-major 2 x 3
        store.stores["f"] = {{0.25f, 0.25f}, Shape(2, 1)};
        const auto merged = SavedFormat::id("w")
                                .transform([](const WeightStore& st, std::vector<float> w) {
                                    const auto& f = st.get("f").values;
                                    for (size_t i = 0; i < w.size(); i++) w[i] += f[i % f.size()];
                                    return w;
                                })
                                .round()
                                .quantise<int16_t>(2);
        // (w + f) * 2 = 1.5, -0.5, 1, 2.5, -1.5, 0.7 -> half away from zero
        const auto mb = merged.write_to_byte_buffer(store);
        const int16_t want_m[6] = {2, -1, 1, 3, -2, 1};
        EXPECT(mb.size() == 12 && !std::memcmp(mb.data(), want_m, 12));
        const auto tb = SavedFormat::id("w").quantise<int8_t>(4).transpose().write_to_byte_buffer(store);
        const int8_t want_t[6] = {2, 1, -4, -2, 4, 0};  // rows (0.5, 0.25, -1), (-0.5, 1, 0.1) x 4, truncated
        EXPECT(tb.size() == 6 && !std::memcmp(tb.data(), want_t, 6));
        const auto all = to_quantised_buffer(store, {SavedFormat::custom({'h', 'd'}), merged, SavedFormat::id("f")}, true);
        EXPECT(all.size() == 64 && all[0] == 'h' && all[14] == 0 && all[17] == 0x3e);  // 2 + 12 + 8 bytes, then padding
        EXPECT(!std::memcmp(all.data() + 22, "bulletbulletbulletbulletbulletbulletbullet", 42));
        auto misuse = [](const std::function<void()>& f, const char* needle) {
            try {
                f();
            } catch (const std::logic_error& e) {
                return std::strstr(e.what(), needle) != nullptr;
            }
            return false;
        };
        EXPECT(misuse([] { SavedFormat::custom({1}).round(); }, "custom"));
        EXPECT(misuse([] { SavedFormat::empty().transpose(); }, "weight id"));
        bool overflow = false;
        try {
            SavedFormat::id("w").quantise<int8_t>(200).write_to_byte_buffer(store);
        } catch (const std::runtime_error& e) {
            overflow = std::strstr(e.what(), "Failed quantisation from f32 to i8!") != nullptr;
        }
        EXPECT(overflow);
    }
    if (argc > 1 && !std::strcmp(argv[1], "gpu")) {
        // one training step of a small bucketed pairwise net on a fixed pseudo-random batch
        const int B = 256, H = 128, NNZ = 32;
        ModelNode stm = b.sparse_input("stm", 12288, NNZ), ntm = b.sparse_input("nstm", 12288, NNZ);
        ModelNode buckets = b.sparse_input("buckets", 8, 1);
        RecognisedNet r = recognise(multi_layer_net(b, stm, ntm, buckets, H, true), 768, B);
        Trainer t(r);
        unsigned long long state = 88172645463325252ull;
        auto rnd = [&] { state ^= state << 13, state ^= state >> 7, state ^= state << 17; return state; };
        auto uni = [&] { return (float)((rnd() >> 11) * (1.0 / 9007199254740992.0)); };
        const auto names = r.abi_names();
        for (size_t i = 0; i < names.size(); i++) {
            int64_t n = 0;
            b200_net_tensor_size(t.handle(), names[i].c_str(), &n);
            std::vector<float> w((size_t)n);
            const float lim = names[i] == "l0w" ? 0.3f : names[i].back() == 'w' ? 0.25f : 0.05f;
            for (auto& v : w) v = (2.f * uni() - 1.f) * lim;
            t.load_weights(r.weight_ids[i], w);
        }
        std::vector<int32_t> s(B * NNZ, -1), n(B * NNZ, -1), k(B);
        std::vector<float> target(B);
        for (int p = 0; p < B; p++) {
            const int cnt = 2 + (int)(rnd() % 31), kb_s = (int)(rnd() % 16), kb_n = (int)(rnd() % 16);
            for (int j = 0; j < cnt; j++) {
                s[p * NNZ + j] = 768 * kb_s + (int)(rnd() % 768);
                n[p * NNZ + j] = 768 * kb_n + (int)(rnd() % 768);
            }
            k[p] = (cnt - 2) / 4;
            target[p] = uni();
        }
        t.set_params_for_weight("l0w", AdamWParams{0.01f, 0.9f, 0.999f, -0.99f, 0.99f});
        t.upload(0, s.data(), n.data(), k.data(), target.data(), B);
        const float first = t.step(0, B, 1e-3f);
        t.upload(1, s.data(), n.data(), k.data(), target.data(), B);
        const float second = t.step(1, B, 1e-3f);
        const std::vector<float> outs = t.eval(1, B);
        std::printf("loss %.9g %.9g out0 %.9g\n", first, second, outs[0]);
        EXPECT(std::isfinite(first) && second < first);
        {   // export: the example's closure (3_input_buckets.rs:46-53) against the library's built-in merge
            const std::vector<SavedFormat> fmt = {
                SavedFormat::id("l0w")
                    .transform([](const WeightStore& st, std::vector<float> w) {
                        const auto& f = st.get("l0f").values;
                        for (size_t i = 0; i < w.size(); i++) w[i] = w[i] + f[i % f.size()];
                        return w;
                    })
                    .round()
                    .quantise<int16_t>(255),
                SavedFormat::id("l0b").round().quantise<int16_t>(255),
                SavedFormat::id("l1w").transpose().round().quantise<int8_t>(64),
                SavedFormat::id("l1b"),
            };
            const auto ours = to_quantised_buffer(t.cpu_weights(), fmt, true);
            b200_saved_format c[4] = {};
            c[0].id = "l0w", c[0].quant = B200_QUANT_I16, c[0].multiplier = 255, c[0].round = 1, c[0].merge_factoriser = 1;
            c[1].id = "l0b", c[1].quant = B200_QUANT_I16, c[1].multiplier = 255, c[1].round = 1;
            c[2].id = "l1w", c[2].quant = B200_QUANT_I8, c[2].multiplier = 64, c[2].round = 1, c[2].transpose = 1;
            c[3].id = "l1b";
            int64_t bytes = 0;
            EXPECT(b200_saved_format_size(t.handle(), c, 4, 1, &bytes) == 0 && bytes == (int64_t)ours.size() && bytes % 64 == 0);
            std::vector<uint8_t> lib((size_t)bytes);
            EXPECT(b200_saved_format_write(t.handle(), c, 4, 1, lib.data(), bytes) == 0 && lib == ours);
            EXPECT(b200_saved_format_write(t.handle(), c, 4, 1, lib.data(), bytes - 1) == B200_ERR_ARG);
        }
        bool threw = false;
        try {
            t.weights("nope");
        } catch (const std::runtime_error&) {
            threw = true;
        }
        EXPECT(threw);
    }
    std::printf(failures ? "%d FAILURES\n" : "ok\n", failures);
    return failures ? 1 : 0;
}
