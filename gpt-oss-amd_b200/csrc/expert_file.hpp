// Packed expert file: the on-disk form of the MoE weights this library consumes.
//
// The reference's exporter dequantises every MXFP4 expert tensor to fp32
// (tools/model_export/gpt-oss-20b/export_model_bin.py:95-133) and its loader
// rounds the fp32 file back to bf16 in 512 MB chunks
// (src/model.cpp:8-56,141-186): 8x the bytes of the checkpoint on disk and a
// conversion on every start.  This file keeps the experts as the checkpoint has
// them -- e2m1 blocks + e8m0 scales + fp32 biases, the arguments of
// moe_b200_set_experts_mxfp4 -- expert-major, one page-aligned record per
// (layer, expert), so that an expert-parallel rank maps and uploads only the
// records of its own shard.  Everything that is not MoE stays in the engine's
// .bin (header and tensor order of src/run.cpp:26-46,196-235); a copy of that
// 15-field header is kept here so that the two files can be checked against
// each other.
//
// Layout (little endian):
//   FileHeader                                   (padded to header_bytes)
//   router section, per layer:   w_router bf16 [E, H], b_router f32 [E]      (padded to 256 B)
//   expert section, [L][E] records of record_bytes (a multiple of 4096) each:
//       blocks1 u8 [2I, H/32, 16]   scales1 u8 [2I, H/32]   bias1 f32 [2I]
//       blocks2 u8 [H,  I/32, 16]   scales2 u8 [H,  I/32]   bias2 f32 [H]
//     (mlp1 rows gate/up interleaved as in the checkpoint, src/run.cpp:667-670;
//      each array starts on a 16-byte boundary inside the record)
//
// Host code only.
#pragma once
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdint>
#include <cstring>
#include <string>

namespace moe {
namespace efile {

constexpr char MAGIC[8] = {'M', 'O', 'E', 'B', '2', '0', '0', '\0'};
constexpr uint32_t VERSION = 1;

// The reference's Config (src/run.cpp:26-46), field for field.
struct RefConfig {
    int32_t vocab_size, hidden_dim, n_experts, experts_per_token, intermediate_dim, n_layers, head_dim,
        n_attn_heads, n_kv_heads, seq_len, initial_context_length;
    float rope_theta, rope_scaling_factor;
    int32_t sliding_window;
    float swiglu_limit;
};
static_assert(sizeof(RefConfig) == 60, "15 four-byte fields");

struct FileHeader {
    char magic[8];
    uint32_t version;
    uint32_t header_bytes;  // offset of the router section
    RefConfig config;
    uint32_t reserved;
    uint64_t router_offset, router_layer_bytes;  // per layer: w_router then b_router, padded
    uint64_t expert_offset, record_bytes;        // [L][E] records
    uint64_t file_bytes;
};

inline uint64_t round_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

// Byte offsets of the six arrays inside a record, and the record size.
struct RecordLayout {
    uint64_t blocks1, scales1, bias1, blocks2, scales2, bias2, bytes;
};
inline RecordLayout record_layout(int H, int I) {
    RecordLayout r{};
    uint64_t o = 0;
    r.blocks1 = o;
    o = round_up(o + (uint64_t)2 * I * (H / 32) * 16, 16);
    r.scales1 = o;
    o = round_up(o + (uint64_t)2 * I * (H / 32), 16);
    r.bias1 = o;
    o = round_up(o + (uint64_t)2 * I * 4, 16);
    r.blocks2 = o;
    o = round_up(o + (uint64_t)H * (I / 32) * 16, 16);
    r.scales2 = o;
    o = round_up(o + (uint64_t)H * (I / 32), 16);
    r.bias2 = o;
    o = round_up(o + (uint64_t)H * 4, 16);
    r.bytes = round_up(o, 4096);
    return r;
}
inline uint64_t router_layer_bytes(int H, int E) { return round_up((uint64_t)E * H * 2 + (uint64_t)E * 4, 256); }

// A read-only mapping of a packed expert file.
struct Mapping {
    int fd = -1;
    const unsigned char* base = nullptr;
    uint64_t size = 0;
    FileHeader hdr{};

    ~Mapping() { close(); }
    void close() {
        if (base)
            munmap(const_cast<unsigned char*>(base), size);
        if (fd >= 0)
            ::close(fd);
        base = nullptr;
        fd = -1;
    }
};

// Opens, maps and validates.  Returns an empty string on success, else what is wrong.
inline std::string open_file(const char* path, Mapping& m) {
    m.fd = ::open(path, O_RDONLY);
    if (m.fd < 0)
        return std::string("cannot open ") + path;
    struct stat st;
    if (fstat(m.fd, &st) != 0 || st.st_size < (off_t)sizeof(FileHeader))
        return std::string(path) + ": too short to be a packed expert file";
    m.size = (uint64_t)st.st_size;
    void* p = mmap(nullptr, m.size, PROT_READ, MAP_PRIVATE, m.fd, 0);
    if (p == MAP_FAILED)
        return std::string("mmap failed for ") + path;
    m.base = static_cast<const unsigned char*>(p);
    memcpy(&m.hdr, m.base, sizeof(FileHeader));
    const FileHeader& h = m.hdr;
    if (memcmp(h.magic, MAGIC, 8) != 0)
        return std::string(path) + ": not a packed expert file (bad magic)";
    if (h.version != VERSION)
        return std::string(path) + ": unsupported file version " + std::to_string(h.version);
    const RefConfig& c = h.config;
    if (c.hidden_dim <= 0 || c.hidden_dim % 64 || c.intermediate_dim <= 0 || c.intermediate_dim % 64 ||
        c.n_experts <= 0 || c.n_layers <= 0 || c.experts_per_token <= 0)
        return std::string(path) + ": implausible dimensions in the header";
    const RecordLayout rl = record_layout(c.hidden_dim, c.intermediate_dim);
    if (h.record_bytes != rl.bytes || h.router_layer_bytes != router_layer_bytes(c.hidden_dim, c.n_experts) ||
        h.router_offset != h.header_bytes || h.header_bytes < sizeof(FileHeader) ||
        h.expert_offset != round_up(h.router_offset + h.router_layer_bytes * (uint64_t)c.n_layers, 4096) ||
        h.file_bytes != h.expert_offset + h.record_bytes * (uint64_t)c.n_layers * (uint64_t)c.n_experts)
        return std::string(path) + ": section offsets do not match the dimensions in the header";
    if (m.size < h.file_bytes)
        return std::string(path) + ": truncated (" + std::to_string(m.size) + " of " +
               std::to_string(h.file_bytes) + " bytes)";
    return std::string();
}

inline const unsigned char* router_of(const Mapping& m, int layer) {
    return m.base + m.hdr.router_offset + m.hdr.router_layer_bytes * (uint64_t)layer;
}
inline const unsigned char* record_of(const Mapping& m, int layer, int expert) {
    return m.base + m.hdr.expert_offset +
           m.hdr.record_bytes * ((uint64_t)layer * (uint64_t)m.hdr.config.n_experts + (uint64_t)expert);
}

}  // namespace efile
}  // namespace moe
