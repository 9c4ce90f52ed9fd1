// GGUF expert tensors -> the resident expert table (host code).
//
// Reference: crates/denno-engine/src/gguf.rs (container reader, v2/v3, split files: :163-330, header
// :795-870), model/qwen4exp.rs:1915-1963 (ExpertW::load: a 3-d tensor ne = [n_in, n_out, n_expert] whose
// bytes are used in place), :1018-1025 (tensor names and shapes of a MoE layer), model/moe_expert.rs:
// 49-82 (ExpertSlice).  There the tensors stay in the file mapping and an LRU moves experts between SSD,
// RAM and VRAM (expert_vram.rs); here a layer's tensors are read from the mapping once and copied into
// HBM, where every expert stays -- and with an expert shard set (dnb_moe_set_expert_shard) a rank copies
// only the byte range of its own experts, which is contiguous because the tensor is expert-major.
//
// The container: magic "GGUF", version (2 or 3), tensor count, key/value count; key/value pairs (string
// key, type tag, value; arrays carry an element type and a count); tensor infos (name, n_dims, dims,
// ggml type, offset relative to the data section); the data section starts at the next multiple of
// general.alignment (default 32).  A split model is several such files with split.no / split.count /
// split.tensors.count; the tensor tables are concatenated in split.no order and metadata is taken from
// part 0 first.
#include <fcntl.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <map>
#include <string>
#include <vector>

#include "dnb_common.cuh"

namespace dnb {

struct GgufTensor {
    std::string name;
    int n_dims = 0;
    uint64_t dims[4] = {1, 1, 1, 1};
    int type = -1;
    uint64_t rel = 0;    // offset inside the part's data section
    int part = 0;
    uint64_t abs = 0;    // offset inside the part's file
    uint64_t nbytes = 0;
};

struct GgufMeta {  // scalar metadata only (arrays are skipped): kept as both views
    bool is_float = false, is_string = false;
    uint64_t u = 0;
    double f = 0.0;
    std::string s;
};

struct GgufPart {
    std::string path;
    const uint8_t* map = nullptr;
    size_t size = 0;
    uint64_t data_start = 0;
    uint64_t split_no = 0, split_count = 0, split_tensors = 0;
    bool has_split = false;
    std::vector<GgufTensor> tensors;
    std::map<std::string, GgufMeta> meta;
};

}  // namespace dnb

struct dnb_gguf {
    std::vector<dnb::GgufPart> parts;
    std::map<std::string, dnb::GgufTensor> tensors;
    std::vector<std::string> order;
    std::map<std::string, dnb::GgufMeta> meta;
};

namespace dnb {

// bytes of a tensor of `type` with these dims, or 0 when the type is unknown here / the row is not whole blocks
static uint64_t gguf_tensor_bytes(int type, const uint64_t* dims, int n_dims) {
    uint64_t n = 1;
    for (int i = 0; i < n_dims; ++i) n *= dims[i];
    if (type == 0) return n * 4;   // F32
    if (type == 1) return n * 2;   // F16
    if (type == 30) return n * 2;  // BF16
    const int be = block_elems(type), ts = type_size(type);
    if (be == 0 || ts == 0 || dims[0] % (uint64_t)be) return 0;
    return n / be * ts;
}

struct Cursor {
    const uint8_t* b;
    size_t n, p = 0;
    bool ok = true;
    template <typename T>
    T rd() {
        T v{};
        if (p + sizeof(T) > n) { ok = false; return v; }
        memcpy(&v, b + p, sizeof(T));
        p += sizeof(T);
        return v;
    }
    std::string str() {
        const uint64_t len = rd<uint64_t>();
        if (!ok || len > n - p) { ok = false; return std::string(); }
        std::string s((const char*)b + p, (size_t)len);
        p += (size_t)len;
        return s;
    }
};

// gguf.h enum gguf_type
enum { GT_U8, GT_I8, GT_U16, GT_I16, GT_U32, GT_I32, GT_F32, GT_BOOL, GT_STRING, GT_ARRAY, GT_U64, GT_I64, GT_F64 };

static bool read_scalar(Cursor& c, uint32_t ty, GgufMeta* m) {
    GgufMeta tmp;
    GgufMeta& o = m ? *m : tmp;
    switch (ty) {
        case GT_U8: o.u = c.rd<uint8_t>(); break;
        case GT_I8: o.u = (uint64_t)(int64_t)c.rd<int8_t>(); break;
        case GT_U16: o.u = c.rd<uint16_t>(); break;
        case GT_I16: o.u = (uint64_t)(int64_t)c.rd<int16_t>(); break;
        case GT_U32: o.u = c.rd<uint32_t>(); break;
        case GT_I32: o.u = (uint64_t)(int64_t)c.rd<int32_t>(); break;
        case GT_BOOL: o.u = c.rd<uint8_t>() ? 1 : 0; break;
        case GT_U64: o.u = c.rd<uint64_t>(); break;
        case GT_I64: o.u = (uint64_t)c.rd<int64_t>(); break;
        case GT_F32: o.f = c.rd<float>(); o.is_float = true; break;
        case GT_F64: o.f = c.rd<double>(); o.is_float = true; break;
        case GT_STRING: o.s = c.str(); o.is_string = true; break;
        default: return false;
    }
    if (o.is_float) o.u = (uint64_t)o.f; else if (!o.is_string) o.f = (double)(int64_t)o.u;
    return c.ok;
}

static int parse_part(GgufPart& P) {
    Cursor c{P.map, P.size};
    if (c.rd<uint32_t>() != 0x46554747u) {
        set_error("gguf: %s: bad magic (not a GGUF file)", P.path.c_str());
        return DNB_ERR_ARG;
    }
    const uint32_t version = c.rd<uint32_t>();
    if (version != 2 && version != 3) {
        set_error("gguf: %s: version %u is not handled (2 and 3 are)", P.path.c_str(), version);
        return DNB_DECLINED;
    }
    const uint64_t n_tensors = c.rd<uint64_t>(), n_kv = c.rd<uint64_t>();
    if (!c.ok || n_tensors > (1u << 24) || n_kv > (1u << 24)) {
        set_error("gguf: %s: implausible header", P.path.c_str());
        return DNB_ERR_ARG;
    }
    uint64_t alignment = 32;
    for (uint64_t i = 0; i < n_kv; ++i) {
        const std::string key = c.str();
        const uint32_t ty = c.rd<uint32_t>();
        if (!c.ok) break;
        if (ty == GT_ARRAY) {
            const uint32_t ety = c.rd<uint32_t>();
            const uint64_t cnt = c.rd<uint64_t>();
            for (uint64_t j = 0; j < cnt && c.ok; ++j)
                if (!read_scalar(c, ety, nullptr)) { c.ok = false; break; }
        } else {
            GgufMeta m;
            if (!read_scalar(c, ty, &m)) { c.ok = false; break; }
            P.meta[key] = m;
        }
    }
    if (!c.ok) {
        set_error("gguf: %s: metadata runs past the end of the file", P.path.c_str());
        return DNB_ERR_ARG;
    }
    auto kv = [&](const char* k, uint64_t* v) {
        auto it = P.meta.find(k);
        if (it == P.meta.end() || it->second.is_string) return false;
        *v = it->second.u;
        return true;
    };
    kv("general.alignment", &alignment);
    if (alignment == 0 || (alignment & (alignment - 1))) {
        set_error("gguf: %s: general.alignment=%llu is not a power of two", P.path.c_str(), (unsigned long long)alignment);
        return DNB_ERR_ARG;
    }
    P.has_split = kv("split.no", &P.split_no) && kv("split.count", &P.split_count);
    kv("split.tensors.count", &P.split_tensors);
    P.tensors.resize((size_t)n_tensors);
    for (auto& t : P.tensors) {
        t.name = c.str();
        t.n_dims = (int)c.rd<uint32_t>();
        if (!c.ok || t.n_dims < 1 || t.n_dims > 4) { c.ok = false; break; }
        for (int d = 0; d < t.n_dims; ++d) t.dims[d] = c.rd<uint64_t>();
        t.type = (int)c.rd<uint32_t>();
        t.rel = c.rd<uint64_t>();
    }
    if (!c.ok) {
        set_error("gguf: %s: tensor table runs past the end of the file", P.path.c_str());
        return DNB_ERR_ARG;
    }
    P.data_start = (c.p + alignment - 1) / alignment * alignment;
    for (auto& t : P.tensors) {
        t.abs = P.data_start + t.rel;
        t.nbytes = gguf_tensor_bytes(t.type, t.dims, t.n_dims);
        // a type this library has no layout for still gets an entry (nbytes 0): it cannot be loaded, only listed
        if (t.nbytes && (t.abs > P.size || t.nbytes > P.size - t.abs)) {
            set_error("gguf: %s: tensor %s reaches past the end of the file", P.path.c_str(), t.name.c_str());
            return DNB_ERR_ARG;
        }
    }
    return DNB_OK;
}

static void gguf_free(dnb_gguf* g) {
    if (!g) return;
    for (auto& P : g->parts)
        if (P.map) munmap((void*)P.map, P.size);
    delete g;
}

}  // namespace dnb

using namespace dnb;

extern "C" {

int dnb_gguf_open(const char* const* paths, int n_paths, dnb_gguf** out) {
    if (!paths || n_paths < 1 || !out) return DNB_ERR_ARG;
    *out = nullptr;
    dnb_gguf* g = new dnb_gguf();
    g->parts.resize(n_paths);
    for (int i = 0; i < n_paths; ++i) {
        GgufPart& P = g->parts[i];
        P.path = paths[i] ? paths[i] : "";
        const int fd = open(P.path.c_str(), O_RDONLY);
        struct stat st;
        if (fd < 0 || fstat(fd, &st) != 0 || st.st_size < 24) {
            if (fd >= 0) close(fd);
            set_error("gguf: cannot open %s", P.path.c_str());
            gguf_free(g);
            return DNB_ERR_ARG;
        }
        P.size = (size_t)st.st_size;
        void* m = mmap(nullptr, P.size, PROT_READ, MAP_PRIVATE, fd, 0);
        close(fd);
        if (m == MAP_FAILED) {
            P.map = nullptr;
            set_error("gguf: cannot map %s", P.path.c_str());
            gguf_free(g);
            return DNB_ERR_ARG;
        }
        P.map = (const uint8_t*)m;
        const int rc = parse_part(P);
        if (rc) {
            gguf_free(g);
            return rc;
        }
    }
    // split files: order by split.no, which must be 0 .. count-1 without gaps, count = number of paths given
    // (gguf.rs:205-245); a single file needs no split keys
    if (n_paths > 1) {
        for (auto& P : g->parts)
            if (!P.has_split) {
                set_error("gguf: %s has no split.no / split.count but %d files were given", P.path.c_str(), n_paths);
                gguf_free(g);
                return DNB_ERR_ARG;
            }
        std::sort(g->parts.begin(), g->parts.end(), [](const GgufPart& a, const GgufPart& b) { return a.split_no < b.split_no; });
        for (int i = 0; i < n_paths; ++i)
            if (g->parts[i].split_no != (uint64_t)i || g->parts[i].split_count != (uint64_t)n_paths) {
                set_error("gguf: split parts are not 0..%d of %d (part %d says no=%llu count=%llu)", n_paths - 1, n_paths, i,
                          (unsigned long long)g->parts[i].split_no, (unsigned long long)g->parts[i].split_count);
                gguf_free(g);
                return DNB_ERR_ARG;
            }
    }
    size_t total = 0;
    for (int i = 0; i < n_paths; ++i) {
        for (auto& t : g->parts[i].tensors) {
            t.part = i;
            if (g->tensors.count(t.name)) {
                set_error("gguf: tensor %s appears twice", t.name.c_str());
                gguf_free(g);
                return DNB_ERR_ARG;
            }
            g->tensors[t.name] = t;
            g->order.push_back(t.name);
            ++total;
        }
        for (auto& kv : g->parts[i].meta)
            if (!g->meta.count(kv.first)) g->meta[kv.first] = kv.second;  // part 0 first, later parts only fill gaps
    }
    if (n_paths > 1 && g->parts[0].split_tensors && g->parts[0].split_tensors != total) {
        set_error("gguf: split.tensors.count=%llu but the parts hold %zu tensors", (unsigned long long)g->parts[0].split_tensors, total);
        gguf_free(g);
        return DNB_ERR_ARG;
    }
    *out = g;
    return DNB_OK;
}

void dnb_gguf_close(dnb_gguf* g) { gguf_free(g); }

int dnb_gguf_n_tensors(const dnb_gguf* g) { return g ? (int)g->order.size() : 0; }

const char* dnb_gguf_tensor_name(const dnb_gguf* g, int index) {
    if (!g || index < 0 || index >= (int)g->order.size()) return nullptr;
    return g->order[index].c_str();
}

int dnb_gguf_tensor_info(const dnb_gguf* g, const char* name, int* ggml_type, int* n_dims, uint64_t dims[4], int* part,
                         uint64_t* file_offset, uint64_t* nbytes) {
    if (!g || !name) return DNB_ERR_ARG;
    auto it = g->tensors.find(name);
    if (it == g->tensors.end()) return DNB_DECLINED;
    const GgufTensor& t = it->second;
    if (ggml_type) *ggml_type = t.type;
    if (n_dims) *n_dims = t.n_dims;
    if (dims) for (int d = 0; d < 4; ++d) dims[d] = t.dims[d];
    if (part) *part = t.part;
    if (file_offset) *file_offset = t.abs;
    if (nbytes) *nbytes = t.nbytes;
    return DNB_OK;
}

const void* dnb_gguf_tensor_data(const dnb_gguf* g, const char* name, uint64_t* nbytes) {
    if (!g || !name) return nullptr;
    auto it = g->tensors.find(name);
    if (it == g->tensors.end() || it->second.nbytes == 0) return nullptr;
    if (nbytes) *nbytes = it->second.nbytes;
    return g->parts[it->second.part].map + it->second.abs;
}

int dnb_gguf_meta_u64(const dnb_gguf* g, const char* key, uint64_t* v) {
    if (!g || !key || !v) return DNB_ERR_ARG;
    auto it = g->meta.find(key);
    if (it == g->meta.end() || it->second.is_string) return DNB_DECLINED;
    *v = it->second.u;
    return DNB_OK;
}

int dnb_gguf_meta_f64(const dnb_gguf* g, const char* key, double* v) {
    if (!g || !key || !v) return DNB_ERR_ARG;
    auto it = g->meta.find(key);
    if (it == g->meta.end() || it->second.is_string) return DNB_DECLINED;
    *v = it->second.f;
    return DNB_OK;
}

int dnb_gguf_meta_str(const dnb_gguf* g, const char* key, char* buf, size_t cap) {
    if (!g || !key || !buf || cap == 0) return DNB_ERR_ARG;
    auto it = g->meta.find(key);
    if (it == g->meta.end() || !it->second.is_string) return DNB_DECLINED;
    snprintf(buf, cap, "%s", it->second.s.c_str());
    return DNB_OK;
}

// blk.<gguf_layer>.<suffix> of a MoE layer (qwen4exp.rs:1018-1025) into layer `layer` of the configured model.
int dnb_load_gguf_layer(dnb_ctx* c, const dnb_gguf* g, int layer, int gguf_layer, const char* norm_name) {
    if (!c || !g) return DNB_ERR_ARG;
    const Model& M = c->model;
    if (layer < 0 || layer >= M.n_layer || gguf_layer < 0) {
        set_error("load_gguf_layer: layer %d outside the configured %d layers", layer, M.n_layer);
        return DNB_ERR_ARG;
    }
    char name[160];
    auto find = [&](const char* suffix) -> const GgufTensor* {
        snprintf(name, sizeof(name), "blk.%d.%s", gguf_layer, suffix);
        auto it = g->tensors.find(name);
        return it == g->tensors.end() ? nullptr : &it->second;
    };
    auto data = [&](const GgufTensor* t) { return g->parts[t->part].map + t->abs; };
    // routed experts: ne = [n_in, n_out, n_expert], expert-major bytes; this rank's experts are one contiguous range
    static const char* const kExp[3] = {"ffn_gate_exps.weight", "ffn_up_exps.weight", "ffn_down_exps.weight"};
    for (int m = 0; m < 3; ++m) {
        const GgufTensor* t = find(kExp[m]);
        if (!t) {
            set_error("load_gguf_layer: %s is missing", name);
            return DNB_DECLINED;
        }
        if (t->n_dims != 3 || (int)t->dims[2] != M.ne || t->nbytes == 0) {
            set_error("load_gguf_layer: %s: expected 3 dims with %d experts in a block format this library decodes", name, M.ne);
            return DNB_DECLINED;
        }
        const size_t eb = (size_t)(t->nbytes / t->dims[2]);
        const int rc = dnb_register_experts(c, layer, m, t->type, (int)t->dims[0], (int)t->dims[1], M.shard_count,
                                            data(t) + (size_t)M.shard_first * eb, eb * (size_t)M.shard_count);
        if (rc) return rc;
    }
    // shared expert (optional): 2-d tensors [n_in, n_out]
    static const char* const kSh[3] = {"ffn_gate_shexp.weight", "ffn_up_shexp.weight", "ffn_down_shexp.weight"};
    const GgufTensor* sh[3] = {find(kSh[0]), find(kSh[1]), find(kSh[2])};
    if (sh[0] && sh[1] && sh[2]) {
        for (int m = 0; m < 3; ++m) {
            const GgufTensor* t = sh[m];
            if (t->n_dims < 2 || t->nbytes == 0) {
                set_error("load_gguf_layer: blk.%d.%s: expected 2 dims in a block format this library decodes", gguf_layer, kSh[m]);
                return DNB_DECLINED;
            }
            const int rc = dnb_register_experts(c, layer, 3 + m, t->type, (int)t->dims[0], (int)t->dims[1], 1, data(t), (size_t)t->nbytes);
            if (rc) return rc;
        }
    }
    // router [n_embd, n_expert] f32, optional bias, optional shared gate row [n_embd] f32, optional norm weight
    const GgufTensor* r = find("ffn_gate_inp.weight");
    if (!r || r->type != 0 || r->n_dims != 2 || (int)r->dims[0] != M.e || (int)r->dims[1] != M.ne) {
        set_error("load_gguf_layer: blk.%d.ffn_gate_inp.weight must be f32 [%d, %d]", gguf_layer, M.e, M.ne);
        return DNB_DECLINED;
    }
    const GgufTensor* bias = find("exp_probs_b.bias");
    const GgufTensor* sgr = find("ffn_gate_inp_shexp.weight");
    const GgufTensor* nw = nullptr;
    if (norm_name && norm_name[0]) nw = find(norm_name);
    if ((bias && (bias->type != 0 || (int)bias->dims[0] != M.ne)) || (sgr && (sgr->type != 0 || (int)sgr->dims[0] != M.e)) ||
        (nw && (nw->type != 0 || (int)nw->dims[0] != M.e)) || (norm_name && norm_name[0] && !nw)) {
        set_error("load_gguf_layer: blk.%d: bias / shared gate row / norm weight must be f32 vectors of the model's sizes", gguf_layer);
        return DNB_DECLINED;
    }
    return dnb_register_router(c, layer, (const float*)data(r), bias ? (const float*)data(bias) : nullptr,
                               nw ? (const float*)data(nw) : nullptr, sgr ? (const float*)data(sgr) : nullptr);
}

}  // extern "C"
