// Weight store: GGUF v3 pack -> one 256-byte aligned device arena of bf16 tensors, and the name
// resolution that turns it into block / forward bindings.  Same structs and entry points as o1.c's
// src/model/weights.h:75-131 (hd_weight_store, hd_weights_to_device_gguf, hd_weight_store_free),
// src/model/block.c:63-100 (hd_block_resolve) and src/model/forward.c:61-111 (hd_forward_resolve).
//
// File -> pinned staging (two 64 MiB slots) -> arena on a dedicated non-blocking stream, so disk
// reads overlap the copies.  BF16 tensors stream through unchanged; F32 / F16 tensors are converted
// to bf16 on the host (RNE) while staging.  Tensor i lands at arena + its own 256-byte aligned offset.
#include "common.cuh"
#include "../../include/o1_b200.h"

#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <string>
#include <vector>

namespace {

char g_werr[512] = {0};
void werr(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_werr, sizeof(g_werr), fmt, ap);
    va_end(ap);
}

struct TensorInfo {
    std::string name;
    std::vector<uint64_t> dims;
    uint32_t type;        // 0 F32, 1 F16, 30 BF16
    uint64_t offset;      // relative to the data section
    uint64_t numel;
};
struct GgufIndex {
    std::vector<TensorInfo> tensors;
    std::vector<std::pair<std::string, std::string>> str_kv;
    uint64_t alignment = 32;
    uint64_t data_start = 0;
};

struct Reader {
    FILE* f;
    bool ok = true;
    template <typename T> T get() {
        T v{};
        if (ok && fread(&v, sizeof(T), 1, f) != 1) ok = false;
        return v;
    }
    std::string str() {
        const uint64_t n = get<uint64_t>();
        if (!ok || n > (1u << 20)) { ok = false; return {}; }
        std::string s(n, '\0');
        if (n && fread(&s[0], 1, n, f) != n) ok = false;
        return s;
    }
    void skip(uint64_t n) { if (ok && fseeko(f, (off_t)n, SEEK_CUR) != 0) ok = false; }
    bool skip_value(uint32_t t, int depth = 0) {
        switch (t) {
            case 0: case 1: case 7: skip(1); return ok;
            case 2: case 3: skip(2); return ok;
            case 4: case 5: case 6: skip(4); return ok;
            case 10: case 11: case 12: skip(8); return ok;
            case 8: str(); return ok;
            case 9: {
                if (depth > 2) { ok = false; return false; }
                const uint32_t et = get<uint32_t>();
                const uint64_t n = get<uint64_t>();
                for (uint64_t i = 0; i < n && ok; ++i) skip_value(et, depth + 1);
                return ok;
            }
            default: ok = false; return false;
        }
    }
};

bool parse_gguf(const char* path, GgufIndex* out) {
    FILE* f = fopen(path, "rb");
    if (!f) { werr("gguf: cannot open %s", path); return false; }
    Reader r{f};
    const uint32_t magic = r.get<uint32_t>(), version = r.get<uint32_t>();
    const uint64_t n_tensors = r.get<uint64_t>(), n_kv = r.get<uint64_t>();
    if (!r.ok || magic != 0x46554747u) { werr("gguf: bad magic in %s", path); fclose(f); return false; }
    if (version != 3) { werr("gguf: unsupported version %u", version); fclose(f); return false; }
    if (n_tensors > (1u << 20) || n_kv > (1u << 16)) { werr("gguf: implausible header counts"); fclose(f); return false; }
    for (uint64_t i = 0; i < n_kv && r.ok; ++i) {
        const std::string key = r.str();
        const uint32_t t = r.get<uint32_t>();
        if (t == 8) out->str_kv.emplace_back(key, r.str());
        else if (t == 4 && key == "general.alignment") out->alignment = r.get<uint32_t>();
        else r.skip_value(t);
    }
    for (uint64_t i = 0; i < n_tensors && r.ok; ++i) {
        TensorInfo ti;
        ti.name = r.str();
        const uint32_t nd = r.get<uint32_t>();
        if (nd > 8) { r.ok = false; break; }
        ti.numel = 1;
        for (uint32_t d = 0; d < nd; ++d) {
            const uint64_t dim = r.get<uint64_t>();
            ti.dims.push_back(dim);
            // element counts beyond 2^40 cannot be real (and their byte size could wrap 64 bits)
            if (dim == 0 || dim > (1ull << 40) || ti.numel > (1ull << 40) / dim) { r.ok = false; break; }
            ti.numel *= dim;
        }
        if (!r.ok) break;
        ti.type = r.get<uint32_t>();
        ti.offset = r.get<uint64_t>();
        if (ti.type != 0 && ti.type != 1 && ti.type != 30) {
            werr("gguf: tensor %s has unsupported type %u (F32, F16, BF16 only)", ti.name.c_str(), ti.type);
            fclose(f);
            return false;
        }
        out->tensors.push_back(std::move(ti));
    }
    if (!r.ok || out->alignment == 0) { werr("gguf: truncated or malformed header in %s", path); fclose(f); return false; }
    const uint64_t pos = (uint64_t)ftello(f);
    out->data_start = (pos + out->alignment - 1) / out->alignment * out->alignment;
    // every tensor's payload must lie inside the file: a truncated pack or a corrupt offset fails here,
    // before any device memory is sized from the header
    uint64_t file_bytes = 0;
    if (fseeko(f, 0, SEEK_END) == 0) file_bytes = (uint64_t)ftello(f);
    fclose(f);
    for (const TensorInfo& t : out->tensors) {
        const uint64_t bytes = t.numel * (t.type == 0 ? 4u : 2u);
        if (t.offset > file_bytes || out->data_start > file_bytes - t.offset ||
            bytes > file_bytes - t.offset - out->data_start) {
            werr("gguf: tensor %s (%llu bytes at offset %llu) lies outside %s (%llu bytes)", t.name.c_str(),
                 (unsigned long long)bytes, (unsigned long long)(out->data_start + t.offset), path,
                 (unsigned long long)file_bytes);
            return false;
        }
    }
    return true;
}

inline uint16_t f16_to_bf16(uint16_t h) {
    const uint32_t sign = (uint32_t)(h >> 15) << 31, exp = (h >> 10) & 0x1f, man = h & 0x3ff;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {
            uint32_t e = 127 - 15 + 1, m = man;
            while (!(m & 0x400)) { m <<= 1; --e; }
            bits = sign | (e << 23) | ((m & 0x3ff) << 13);
        }
    } else if (exp == 0x1f) bits = sign | 0x7f800000u | (man << 13);
    else bits = sign | ((exp - 15 + 127) << 23) | (man << 13);
    float f;
    memcpy(&f, &bits, 4);
    return o1::f32_to_bf16(f);
}

const void* find_tensor(const hd_weight_store* ws, const char* name) {
    for (int64_t i = 0; i < ws->n_allocs; ++i)
        if (ws->allocs[i].name[0] && strcmp(ws->allocs[i].name, name) == 0) return ws->allocs[i].dev_ptr;
    return nullptr;
}

}  // namespace

extern "C" {

const char* hd_weights_last_error(void) { return g_werr; }

// Header-only parse (no GPU): number of tensors, or -1.  name/numel/type of tensor i through the getters.
int64_t o1_gguf_probe(const char* path, int64_t index, char* name_out, size_t name_cap, int64_t* numel,
                      int* type, int64_t* file_offset) {
    GgufIndex idx;
    if (!path || !parse_gguf(path, &idx)) return -1;
    if (index >= 0 && index < (int64_t)idx.tensors.size()) {
        const TensorInfo& t = idx.tensors[index];
        if (name_out && name_cap) snprintf(name_out, name_cap, "%s", t.name.c_str());
        if (numel) *numel = (int64_t)t.numel;
        if (type) *type = (int)t.type;
        if (file_offset) *file_offset = (int64_t)(idx.data_start + t.offset);
    }
    return (int64_t)idx.tensors.size();
}

static hd_status load_gguf(const char* gguf_path, int device_id, hd_weight_store* out, bool payload);

hd_status hd_weights_to_device_gguf(const char* gguf_path, int device_id, hd_weight_store* out) {
    return load_gguf(gguf_path, device_id, out, true);
}
// Same store (arena allocated, every tensor's address fixed by the header) without reading the payload: the
// caller fills the arena from another rank's copy (one disk read + a broadcast over NVLink instead of one
// disk read per GPU).  The arena layout depends only on the header, so it is identical on every rank.
hd_status o1_weights_gguf_layout(const char* gguf_path, int device_id, hd_weight_store* out) {
    return load_gguf(gguf_path, device_id, out, false);
}

static hd_status load_gguf(const char* gguf_path, int device_id, hd_weight_store* out, bool payload) {
    if (!gguf_path || !out) { werr("weights: null argument"); return HD_ERR_MISSING; }
    memset(out, 0, sizeof(*out));
    GgufIndex idx;
    if (!parse_gguf(gguf_path, &idx)) return HD_ERR_PARSE;
    if (idx.tensors.empty()) { werr("weights: %s holds no tensors", gguf_path); return HD_ERR_MANIFEST; }
    cudaError_t e = cudaSetDevice(device_id);
    cudaDeviceProp prop;
    if (e == cudaSuccess) e = cudaGetDeviceProperties(&prop, device_id);
    if (e != cudaSuccess) { werr("weights: device %d: %s", device_id, cudaGetErrorString(e)); return HD_ERR_RUNTIME; }
    out->device_id = device_id;
    snprintf(out->device_name, sizeof(out->device_name), "%s", prop.name);
    out->compute_major = prop.major;
    out->compute_minor = prop.minor;
    out->device_mem_bytes = (int64_t)prop.totalGlobalMem;

    const size_t n = idx.tensors.size();
    // A pack of BF16 tensors at 256-byte aligned offsets keeps the file's own layout, as the reference's loader
    // does (src/model/weights.c:536-650: arena = payload bytes, tensor i at arena + its file offset), so a host
    // that addresses tensors by offset finds them where it expects.  Packs with F32 / F16 tensors (converted to
    // bf16 here, half or equal size) or unaligned offsets are laid out cumulatively instead.
    std::vector<uint64_t> arena_off(n);
    uint64_t total = 0;
    bool file_layout = true;
    for (size_t i = 0; i < n; ++i)
        if (idx.tensors[i].type != 30 || (idx.tensors[i].offset & 255)) file_layout = false;
    if (file_layout) {
        for (size_t i = 0; i < n; ++i) {
            arena_off[i] = idx.tensors[i].offset;
            total = std::max<uint64_t>(total, idx.tensors[i].offset + idx.tensors[i].numel * 2);
        }
        total = (total + 255) & ~(uint64_t)255;
    } else {
        for (size_t i = 0; i < n; ++i) {
            arena_off[i] = total;
            total += (idx.tensors[i].numel * 2 + 255) & ~(uint64_t)255;
        }
    }
    out->allocs = (hd_device_alloc*)calloc(n, sizeof(hd_device_alloc));
    if (!out->allocs) { werr("weights: out of host memory"); return HD_ERR_OOM; }
    e = cudaMalloc(&out->arena_ptr, total);
    if (e != cudaSuccess) {
        werr("weights: cudaMalloc of %llu bytes: %s", (unsigned long long)total, cudaGetErrorString(e));
        free(out->allocs); out->allocs = nullptr;
        return HD_ERR_OOM;
    }
    // the gaps between tensors hold zeros, as in a pack's padded payload (the reference's loader copies the
    // payload whole, src/model/weights.c:566-612)
    if (cudaMemset(out->arena_ptr, 0, total) != cudaSuccess) {
        werr("weights: clearing the arena failed");
        cudaFree(out->arena_ptr); out->arena_ptr = nullptr;
        free(out->allocs); out->allocs = nullptr;
        return HD_ERR_RUNTIME;
    }
    out->arena_bytes = (int64_t)total;
    out->device_bytes_allocated = (int64_t)total;
    out->n_allocations = 1;
    out->n_allocs = (int64_t)n;

    const size_t SLOT = 64u << 20;
    uint8_t* pinned[2] = {nullptr, nullptr};
    cudaEvent_t done[2] = {nullptr, nullptr};
    cudaStream_t st = nullptr;
    FILE* f = fopen(gguf_path, "rb");
    std::vector<uint8_t> raw;
    hd_status rc = HD_OK;
    if (!f) { werr("weights: cannot open %s", gguf_path); rc = HD_ERR_IO; }
    if (rc == HD_OK && (cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) != cudaSuccess ||
                        cudaMallocHost(&pinned[0], SLOT) != cudaSuccess || cudaMallocHost(&pinned[1], SLOT) != cudaSuccess ||
                        cudaEventCreate(&done[0]) != cudaSuccess || cudaEventCreate(&done[1]) != cudaSuccess)) {
        werr("weights: staging set-up failed");
        rc = HD_ERR_OOM;
    }
    int slot = 0;
    bool used[2] = {false, false};
    for (size_t i = 0; i < n && rc == HD_OK; ++i) {
        const TensorInfo& t = idx.tensors[i];
        hd_device_alloc& a = out->allocs[i];
        a.dev_ptr = (uint8_t*)out->arena_ptr + arena_off[i];
        a.nbytes = (int64_t)(t.numel * 2);
        snprintf(a.name, sizeof(a.name), "%s", t.name.c_str());
        if ((int64_t)t.numel > out->largest_numel) {
            out->largest_numel = (int64_t)t.numel;
            snprintf(out->largest_name, sizeof(out->largest_name), "%s", t.name.c_str());
        }
        const size_t esz = t.type == 0 ? 4 : 2;
        if (!payload) continue;
        if (fseeko(f, (off_t)(idx.data_start + t.offset), SEEK_SET) != 0) { werr("weights: seek failed for %s", a.name); rc = HD_ERR_IO; break; }
        uint64_t done_el = 0;
        while (done_el < t.numel && rc == HD_OK) {
            const uint64_t chunk = std::min<uint64_t>(t.numel - done_el, SLOT / 2);
            if (used[slot] && cudaEventSynchronize(done[slot]) != cudaSuccess) { werr("weights: staging sync failed"); rc = HD_ERR_RUNTIME; break; }
            uint16_t* dst16 = (uint16_t*)pinned[slot];
            if (t.type == 30) {
                if (fread(dst16, 2, chunk, f) != chunk) { werr("weights: short read in %s", a.name); rc = HD_ERR_IO; break; }
            } else {
                raw.resize(chunk * esz);
                if (fread(raw.data(), esz, chunk, f) != chunk) { werr("weights: short read in %s", a.name); rc = HD_ERR_IO; break; }
                if (t.type == 0) { const float* s = (const float*)raw.data(); for (uint64_t k = 0; k < chunk; ++k) dst16[k] = o1::f32_to_bf16(s[k]); }
                else { const uint16_t* s = (const uint16_t*)raw.data(); for (uint64_t k = 0; k < chunk; ++k) dst16[k] = f16_to_bf16(s[k]); }
            }
            e = cudaMemcpyAsync((uint8_t*)a.dev_ptr + done_el * 2, dst16, chunk * 2, cudaMemcpyHostToDevice, st);
            if (e == cudaSuccess) e = cudaEventRecord(done[slot], st);
            if (e != cudaSuccess) { werr("weights: upload of %s: %s", a.name, cudaGetErrorString(e)); rc = HD_ERR_RUNTIME; break; }
            used[slot] = true;
            slot ^= 1;
            done_el += chunk;
            out->host_bytes_loaded += (int64_t)(chunk * esz);
        }
    }
    if (st && cudaStreamSynchronize(st) != cudaSuccess && rc == HD_OK) { werr("weights: upload stream failed"); rc = HD_ERR_RUNTIME; }
    if (f) fclose(f);
    for (int s = 0; s < 2; ++s) {
        if (pinned[s]) cudaFreeHost(pinned[s]);
        if (done[s]) cudaEventDestroy(done[s]);
    }
    out->upload_stream = st;
    out->gemm = hd_gemm_runtime_init(device_id, 0);
    if (rc != HD_OK) hd_weight_store_free(out);
    return rc;
}

void hd_weight_store_free(hd_weight_store* s) {
    if (!s) return;
    if (s->arena_ptr) cudaFree(s->arena_ptr);
    if (s->upload_stream) cudaStreamDestroy((cudaStream_t)s->upload_stream);
    if (s->gemm) hd_gemm_runtime_destroy(s->gemm);
    free(s->allocs);
    memset(s, 0, sizeof(*s));
}

hd_status hd_block_resolve(const hd_weight_store* wstore, int layer_idx, hd_block_binding* out) {
    if (!wstore || !out) { hd_set_error("block: null argument in resolve"); return HD_ERR_MISSING; }
    static const char* slot[11] = {
        "self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight", "self_attn.o_proj.weight",
        "input_layernorm.weight", "post_attention_layernorm.weight", "mlp.gate_proj.weight", "mlp.up_proj.weight",
        "mlp.down_proj.weight", "self_attn.q_norm.weight", "self_attn.k_norm.weight"};
    const void* p[11];
    char name[256];
    for (int i = 0; i < 11; ++i) {
        snprintf(name, sizeof(name), "model.language_model.layers.%d.%s", layer_idx, slot[i]);
        p[i] = find_tensor(wstore, name);
        if (!p[i]) { hd_set_error("block: missing weight %s", name); return HD_ERR_MISSING; }
    }
    out->layer_idx = layer_idx;
    out->q_proj = p[0]; out->k_proj = p[1]; out->v_proj = p[2]; out->o_proj = p[3];
    out->input_ln = p[4]; out->post_ln = p[5];
    out->gate_proj = p[6]; out->up_proj = p[7]; out->down_proj = p[8];
    out->q_norm = p[9]; out->k_norm = p[10];
    return HD_OK;
}

hd_status hd_forward_resolve(const hd_weight_store* wstore, int n_layers, hd_forward_binding* out) {
    if (!wstore || !out || n_layers <= 0) { hd_set_error("forward: null argument in resolve"); return HD_ERR_MISSING; }
    hd_forward_binding b;
    memset(&b, 0, sizeof(b));
    b.embed_tokens = find_tensor(wstore, "model.language_model.embed_tokens.weight");
    b.te0_w = find_tensor(wstore, "model.t_embedder1.mlp.0.weight");
    b.te0_b = find_tensor(wstore, "model.t_embedder1.mlp.0.bias");
    b.te2_w = find_tensor(wstore, "model.t_embedder1.mlp.2.weight");
    b.te2_b = find_tensor(wstore, "model.t_embedder1.mlp.2.bias");
    b.xe1_w = find_tensor(wstore, "model.x_embedder.proj1.weight");
    b.xe2_w = find_tensor(wstore, "model.x_embedder.proj2.weight");
    b.xe2_b = find_tensor(wstore, "model.x_embedder.proj2.bias");
    b.fl_w = find_tensor(wstore, "model.final_layer2.linear.weight");
    b.fl_b = find_tensor(wstore, "model.final_layer2.linear.bias");
    b.fnorm_w = find_tensor(wstore, "model.language_model.norm.weight");
    if (!b.embed_tokens || !b.te0_w || !b.te0_b || !b.te2_w || !b.te2_b || !b.xe1_w || !b.xe2_w || !b.xe2_b ||
        !b.fl_w || !b.fl_b || !b.fnorm_w) {
        hd_set_error("forward: missing global weight(s) in store");
        return HD_ERR_MISSING;
    }
    b.n_layers = n_layers;
    b.blocks = (hd_block_binding*)calloc((size_t)n_layers, sizeof(hd_block_binding));
    if (!b.blocks) { hd_set_error("forward: oom allocating block bindings"); return HD_ERR_OOM; }
    for (int i = 0; i < n_layers; ++i) {
        const hd_status s = hd_block_resolve(wstore, i, &b.blocks[i]);
        if (s != HD_OK) { hd_forward_binding_free(&b); return s; }
    }
    *out = b;
    return HD_OK;
}

void hd_forward_binding_free(hd_forward_binding* b) {
    if (!b) return;
    free(b->blocks);
    b->blocks = nullptr;
    b->n_layers = 0;
}

}  // extern "C"
