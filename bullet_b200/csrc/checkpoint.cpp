// Checkpoint files in the reference's format, so a run can move between bullet and this
// library in either direction.
//
// Optimiser::write_to_checkpoint (crates/trainer/src/optimiser.rs:218-224) and
// AdamW::write_to_checkpoint (crates/trainer/src/optimiser/adam.rs:300-305) write three files
// into a directory: weights.bin, momentum.bin, velocity.bin.  Each is a sequence of records,
// one per tensor in name order: the ASCII id, '\n', the element count as a little-endian
// u64, then the f32 values little-endian (crates/trainer/src/model/weights.rs:404-467).
// Loading matches records to tensors by id, in any order (adam.rs:307-324).
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/bullet_b200.h"
#include "common.h"

namespace {

// kinds 0, 1, 2, and Ranger's slow weights (ranger.rs:115-134 writes them as slow.bin beside the inner optimiser's files)
const char* const kFiles[4] = {"weights.bin", "momentum.bin", "velocity.bin", "slow.bin"};
const int kKinds[4] = {B200_KIND_WEIGHT, B200_KIND_MOMENTUM, B200_KIND_VELOCITY, B200_KIND_SLOW};
int file_count(b200_net* net) {
    int64_t slow = 0;
    b200_net_get_stat(net, "slow_weights", &slow);
    return slow ? 4 : 3;
}
const char* const kIds[] = {"l0b", "l0f", "l0w", "l1b", "l1w", "l2b", "l2w", "l3b", "l3w"};  // name order

}  // namespace

extern "C" {

int b200_checkpoint_save(b200_net* net, const char* dir) {
    if (!net || !dir) return b200::fail(B200_ERR_ARG, "checkpoint_save: null argument");
    std::vector<float> values;
    const int files = file_count(net);
    for (int kind = 0; kind < files; kind++) {
        const std::string path = std::string(dir) + "/" + kFiles[kind];
        FILE* f = std::fopen(path.c_str(), "wb");
        if (!f) return b200::fail(B200_ERR_ARG, "checkpoint_save: cannot create %s", path.c_str());
        for (const char* id : kIds) {
            int64_t n = 0;
            if (b200_net_tensor_size(net, id, &n) != 0) continue;  // this network has no such tensor
            values.resize((size_t)n);
            if (int rc = b200_net_get_tensor(net, id, kKinds[kind], values.data(), n)) {
                std::fclose(f);
                return rc;
            }
            const uint64_t count = (uint64_t)n;  // the host is little-endian, as is the format
            bool ok = std::fwrite(id, 1, std::strlen(id), f) == std::strlen(id) && std::fputc('\n', f) != EOF &&
                      std::fwrite(&count, sizeof count, 1, f) == 1 &&
                      std::fwrite(values.data(), sizeof(float), values.size(), f) == values.size();
            if (!ok) {
                std::fclose(f);
                return b200::fail(B200_ERR_ARG, "checkpoint_save: short write to %s", path.c_str());
            }
        }
        if (std::fclose(f) != 0) return b200::fail(B200_ERR_ARG, "checkpoint_save: closing %s failed", path.c_str());
    }
    return 0;
}

int b200_checkpoint_load(b200_net* net, const char* dir) {
    if (!net || !dir) return b200::fail(B200_ERR_ARG, "checkpoint_load: null argument");
    // All three files are read and checked (ids, counts, the set of tensors) before anything reaches the
    // device: a truncated or foreign file leaves the network exactly as it was.
    struct Record {
        std::string id;
        size_t at;       // offset of the values inside the file's bytes
        int64_t count;
    };
    std::vector<unsigned char> bytes[4];
    std::vector<Record> records[4];
    const int files = file_count(net);
    for (int kind = 0; kind < files; kind++) {
        const std::string path = std::string(dir) + "/" + kFiles[kind];
        FILE* f = std::fopen(path.c_str(), "rb");
        if (!f) return b200::fail(B200_ERR_ARG, "checkpoint_load: cannot open %s", path.c_str());
        std::fseek(f, 0, SEEK_END);
        const long size = std::ftell(f);
        std::fseek(f, 0, SEEK_SET);
        std::vector<unsigned char>& buf = bytes[kind];
        buf.resize((size_t)std::max(0L, size));
        const bool ok = std::fread(buf.data(), 1, buf.size(), f) == buf.size();
        std::fclose(f);
        if (!ok) return b200::fail(B200_ERR_ARG, "checkpoint_load: short read from %s", path.c_str());
        size_t at = 0;
        while (at < buf.size()) {
            std::string id;
            while (at < buf.size() && buf[at] != '\n') id.push_back((char)buf[at++]);
            if (at + 1 + 8 > buf.size()) return b200::fail(B200_ERR_DATA, "checkpoint_load: %s is truncated after id '%s'", path.c_str(), id.c_str());
            at++;  // the newline
            uint64_t count = 0;
            std::memcpy(&count, buf.data() + at, 8);
            at += 8;
            if (count > (buf.size() - at) / 4) return b200::fail(B200_ERR_DATA, "checkpoint_load: record '%s' of %s runs past the end", id.c_str(), path.c_str());
            int64_t n = 0;
            if (b200_net_tensor_size(net, id.c_str(), &n) != 0)
                return b200::fail(B200_ERR_DATA, "checkpoint_load: %s holds tensor '%s', which this network does not have", path.c_str(), id.c_str());
            if ((uint64_t)n != count)
                return b200::fail(B200_ERR_DATA, "checkpoint_load: tensor '%s' has %lld values here, %llu in %s", id.c_str(), (long long)n,
                                  (unsigned long long)count, path.c_str());
            for (const Record& r : records[kind])
                if (r.id == id) return b200::fail(B200_ERR_DATA, "checkpoint_load: %s holds tensor '%s' twice", path.c_str(), id.c_str());
            records[kind].push_back({id, at, n});
            at += (size_t)count * 4;
        }
        int expected = 0;
        for (const char* id : kIds) {
            int64_t n = 0;
            if (b200_net_tensor_size(net, id, &n) == 0) expected++;
        }
        if ((int)records[kind].size() != expected)
            return b200::fail(B200_ERR_DATA, "checkpoint_load: %s holds %d tensors, the network has %d", path.c_str(), (int)records[kind].size(), expected);
    }
    std::vector<float> values;
    for (int kind = 0; kind < files; kind++)
        for (const Record& r : records[kind]) {
            values.resize((size_t)r.count);
            std::memcpy(values.data(), bytes[kind].data() + r.at, (size_t)r.count * 4);
            if (int rc = b200_net_set_tensor(net, r.id.c_str(), kKinds[kind], values.data(), r.count)) return rc;
        }
    return 0;
}

}  // extern "C"
