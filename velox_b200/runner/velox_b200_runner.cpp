// Stand-alone runner over the C ABI of libvelox_b200: the role of the reference's host runner
// (src/runners/velox_cuda_runner.cu:327-700) with its command line and report lines, for any Llama-style
// decoder shape instead of one compiled-in model.
//
//   velox_b200_runner --weights model.safetensors|model.gguf --tokens 1,2,3 --steps 32 [--quantize f16|q4_0|q4g32|i8]
//                     [--model smollm-135m | --dims vocab,d_model,layers,q_heads,kv_heads,head_dim,ffn]
//                     [--rope-theta T] [--rms-eps E] [--qkv-bias] [--synthetic SEED] [--no-cuda-graph] [--verbose]
//                     [--speculative [K]] [--draft-len K] [--spec-ema X] [--context-len N]
//                     [--temperature T --top-p P [--seed S]]
//
// Weights come from a safetensors file (F32 / F16 / BF16 tensors under the Hugging Face Llama names listed in
// src/runtime.rs:1274-1290; a missing lm_head.weight means tied embeddings), from a GGUF v3 file (F32 / F16 / Q4_K /
// Q6_K tensors under the llama.cpp names the reference's K2 runner reads, src/runners/velox_cuda_runner_k2.cu:1918-1963;
// a missing output.weight falls back to token_embd.weight) or, with --synthetic, from the library's counter-based
// generator.  The speculative flags are the ones `veloxc --run` passes through (src/cli.rs:653-683).  Everything
// numerical happens in the library; this file is host plumbing.
#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include "velox_b200.h"

namespace {

struct TensorInfo {
    int fmt = -1;  // VB_FMT_F32 / F16 / BF16
    std::vector<uint64_t> shape;
    uint64_t begin = 0, end = 0;  // byte range inside the data section
};

// ---- a JSON reader just large enough for a safetensors header ------------------------------------------------
struct Json {
    const char* p;
    const char* e;
    bool ok = true;
    void ws() { while (p < e && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
    bool eat(char c) { ws(); if (p < e && *p == c) { ++p; return true; } return false; }
    std::string str() {
        std::string s;
        ws();
        if (p >= e || *p != '"') { ok = false; return s; }
        for (++p; p < e && *p != '"'; ++p) {
            if (*p == '\\' && p + 1 < e) ++p;  // names and dtypes hold no escapes that matter here
            s.push_back(*p);
        }
        if (p < e) ++p; else ok = false;
        return s;
    }
    uint64_t num() {
        ws();
        uint64_t v = 0;
        bool any = false;
        while (p < e && *p >= '0' && *p <= '9') { v = v * 10 + (uint64_t)(*p - '0'); ++p; any = true; }
        if (!any) ok = false;
        return v;
    }
    void skip() {  // any value
        ws();
        if (p >= e) { ok = false; return; }
        if (*p == '"') { str(); return; }
        if (*p == '{' || *p == '[') {
            const char open = *p, close = open == '{' ? '}' : ']';
            int depth = 0;
            bool in_str = false;
            for (; p < e; ++p) {
                if (in_str) { if (*p == '\\') ++p; else if (*p == '"') in_str = false; continue; }
                if (*p == '"') in_str = true;
                else if (*p == open) ++depth;
                else if (*p == close && --depth == 0) { ++p; return; }
            }
            ok = false;
            return;
        }
        while (p < e && *p != ',' && *p != '}' && *p != ']') ++p;
    }
};

bool parse_header(const char* text, uint64_t n, std::map<std::string, TensorInfo>* out) {
    Json j{text, text + n};
    if (!j.eat('{')) return false;
    if (j.eat('}')) return true;
    do {
        const std::string name = j.str();
        if (!j.ok || !j.eat(':')) return false;
        if (name == "__metadata__") { j.skip(); continue; }
        TensorInfo t;
        if (!j.eat('{')) return false;
        do {
            const std::string key = j.str();
            if (!j.ok || !j.eat(':')) return false;
            if (key == "dtype") {
                const std::string d = j.str();
                t.fmt = d == "F32" ? VB_FMT_F32 : d == "F16" ? VB_FMT_F16 : d == "BF16" ? VB_FMT_BF16 : -1;
            } else if (key == "shape") {
                if (!j.eat('[')) return false;
                if (!j.eat(']')) { do t.shape.push_back(j.num()); while (j.eat(',')); if (!j.eat(']')) return false; }
            } else if (key == "data_offsets") {
                if (!j.eat('[')) return false;
                t.begin = j.num();
                if (!j.eat(',')) return false;
                t.end = j.num();
                if (!j.eat(']')) return false;
            } else {
                j.skip();
            }
        } while (j.ok && j.eat(','));
        if (!j.ok || !j.eat('}')) return false;
        (*out)[name] = t;
    } while (j.eat(','));
    return j.ok && j.eat('}');
}

// ---- GGUF v3 directory (src/runners/velox_cuda_runner_k2.cu:70-178): tensor name -> type, dims, byte range -----------
struct GgufTensor {
    uint32_t type = 0;
    std::vector<uint64_t> dims;  // dims[0] is the innermost (columns)
    uint64_t offset = 0, bytes = 0;
};
bool gguf_skip_value(const unsigned char* base, size_t* pos, size_t size, uint32_t vtype, int depth = 0) {
    auto need = [&](size_t n) { return *pos + n <= size; };
    switch (vtype) {
    case 0: case 1: case 7: if (!need(1)) return false; *pos += 1; return true;
    case 2: case 3: if (!need(2)) return false; *pos += 2; return true;
    case 4: case 5: case 6: if (!need(4)) return false; *pos += 4; return true;
    case 10: case 11: case 12: if (!need(8)) return false; *pos += 8; return true;
    case 8: {
        if (!need(8)) return false;
        uint64_t n;
        memcpy(&n, base + *pos, 8);
        *pos += 8;
        if (n > size - *pos) return false;
        *pos += (size_t)n;
        return true;
    }
    case 9: {
        if (!need(12) || depth > 4) return false;
        uint32_t et;
        uint64_t n;
        memcpy(&et, base + *pos, 4);
        memcpy(&n, base + *pos + 4, 8);
        *pos += 12;
        for (uint64_t i = 0; i < n; ++i)
            if (!gguf_skip_value(base, pos, size, et, depth + 1)) return false;
        return true;
    }
    default: return false;
    }
}
bool parse_gguf(const unsigned char* base, size_t size, std::map<std::string, GgufTensor>* out, size_t* data_start) {
    if (size < 24 || memcmp(base, "GGUF", 4) != 0) return false;
    size_t pos = 4;
    uint32_t version;
    uint64_t n_tensors, n_kv;
    memcpy(&version, base + pos, 4); pos += 4;
    memcpy(&n_tensors, base + pos, 8); pos += 8;
    memcpy(&n_kv, base + pos, 8); pos += 8;
    if (version < 2 || n_tensors > (1u << 20) || n_kv > (1u << 20)) return false;
    for (uint64_t k = 0; k < n_kv; ++k) {
        if (!gguf_skip_value(base, &pos, size, 8)) return false;  // key
        if (pos + 4 > size) return false;
        uint32_t vtype;
        memcpy(&vtype, base + pos, 4); pos += 4;
        if (!gguf_skip_value(base, &pos, size, vtype)) return false;
    }
    for (uint64_t t = 0; t < n_tensors; ++t) {
        if (pos + 8 > size) return false;
        uint64_t nlen;
        memcpy(&nlen, base + pos, 8); pos += 8;
        if (nlen > size - pos) return false;
        const std::string name((const char*)base + pos, (size_t)nlen);
        pos += (size_t)nlen;
        GgufTensor g;
        uint32_t n_dims;
        if (pos + 4 > size) return false;
        memcpy(&n_dims, base + pos, 4); pos += 4;
        if (n_dims > 4 || pos + 8ull * n_dims + 12 > size) return false;
        uint64_t n_elem = 1;
        for (uint32_t d = 0; d < n_dims; ++d) { uint64_t v; memcpy(&v, base + pos, 8); pos += 8; g.dims.push_back(v); n_elem *= v; }
        memcpy(&g.type, base + pos, 4); pos += 4;
        memcpy(&g.offset, base + pos, 8); pos += 8;
        g.bytes = vb_gguf_tensor_bytes((int32_t)g.type, n_elem);
        (*out)[name] = g;
    }
    *data_start = (pos + 31) & ~(size_t)31;  // the reference's fixed 32-byte alignment (:174)
    for (const auto& kv : *out)
        if (kv.second.bytes && (*data_start + kv.second.offset > size || kv.second.bytes > size - *data_start - kv.second.offset)) return false;
    return true;
}

struct Shape { uint32_t vocab, d_model, layers, q_heads, kv_heads, head_dim, ffn; float theta, eps; bool bias; const char* name; };
const Shape kShapes[] = {
    {49152, 576, 30, 9, 3, 64, 1536, 10000.0f, 1e-5f, false, "smollm-135m"},     // examples/tinystories_smollm.vlx
    {128256, 4096, 32, 32, 8, 128, 14336, 500000.0f, 1e-5f, false, "llama3-8b"},  // examples/llama3_8b.vlx
    {152064, 3584, 28, 28, 4, 128, 18944, 1000000.0f, 1e-6f, true, "qwen2.5-7b"}, // examples/qwen2_5_7b.vlx
};

int fail(const char* what) {
    fprintf(stderr, "Error: %s: %s\n", what, vb_last_error());
    return 1;
}

double now_ms() {
    return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

}  // namespace

int main(int argc, char** argv) {
    const char* weights_path = nullptr;
    std::vector<uint32_t> prompt = {1, 2, 3, 4};
    size_t steps = 4;
    bool verbose = false, use_graph = true, synthetic = false;
    uint64_t seed = 1;
    uint32_t weight_fmt = VB_FMT_F32;
    bool speculative = false;
    int draft_len = 3;
    float spec_ema = 0.20f, temperature = 0.0f, top_p = 0.0f;
    size_t context_len = 0;
    uint64_t sample_seed = 0;
    Shape sh = kShapes[0];
    for (int i = 1; i < argc; ++i) {
        const std::string a = argv[i];
        auto next = [&]() -> const char* { return i + 1 < argc ? argv[++i] : ""; };
        if (a == "--weights") weights_path = next();
        else if (a == "--tokens") {
            prompt.clear();
            for (const char* s = next(); *s;) {
                char* end = nullptr;
                const unsigned long v = strtoul(s, &end, 10);
                if (end == s) break;
                prompt.push_back((uint32_t)v);
                s = (*end == ',') ? end + 1 : end;
            }
        } else if (a == "--steps") steps = (size_t)strtoul(next(), nullptr, 10);
        else if (a == "--verbose") verbose = true;
        else if (a == "--no-cuda-graph") use_graph = false;
        else if (a == "--speculative") {  // optional numeric draft width, as the reference runner parses it (:1772-1778)
            speculative = true;
            if (i + 1 < argc && argv[i + 1][0] != '-') { draft_len = atoi(argv[++i]); if (draft_len <= 0) draft_len = 3; if (draft_len > 7) draft_len = 7; }
        } else if (a == "--draft-len") { draft_len = atoi(next()); if (draft_len <= 0) draft_len = 3; if (draft_len > 7) draft_len = 7; }
        else if (a == "--spec-ema") { spec_ema = (float)atof(next()); if (spec_ema < 0.0f) spec_ema = 0.0f; if (spec_ema > 0.95f) spec_ema = 0.95f; }
        else if (a == "--context-len") context_len = (size_t)strtoul(next(), nullptr, 10);
        else if (a == "--temperature") temperature = strtof(next(), nullptr);
        else if (a == "--top-p") top_p = strtof(next(), nullptr);
        else if (a == "--seed") sample_seed = strtoull(next(), nullptr, 10);
        else if (a == "--synthetic") { synthetic = true; seed = strtoull(next(), nullptr, 10); }
        else if (a == "--quantize" || a.rfind("--quantize=", 0) == 0) {
            const std::string q = a == "--quantize" ? std::string(next()) : a.substr(11);
            if (q == "f16" || q == "fp16") weight_fmt = VB_FMT_F16;
            else if (q == "q4_0" || q == "int4" || q == "w4a16") weight_fmt = VB_FMT_Q4G64REF;  // the reference's own int4
            else if (q == "q4g32") weight_fmt = VB_FMT_Q4G32;
            else if (q == "i8" || q == "int8") weight_fmt = VB_FMT_I8PC;
            else if (q == "f32" || q == "fp32") weight_fmt = VB_FMT_F32;
            else { fprintf(stderr, "Error: unknown --quantize '%s'\n", q.c_str()); return 2; }
        } else if (a == "--model") {
            const std::string m = next();
            bool found = false;
            for (const Shape& s : kShapes) if (m == s.name) { sh = s; found = true; }
            if (!found) { fprintf(stderr, "Error: unknown --model '%s'\n", m.c_str()); return 2; }
        } else if (a == "--dims") {
            unsigned v[7];
            if (sscanf(next(), "%u,%u,%u,%u,%u,%u,%u", &v[0], &v[1], &v[2], &v[3], &v[4], &v[5], &v[6]) != 7) {
                fprintf(stderr, "Error: --dims wants vocab,d_model,layers,q_heads,kv_heads,head_dim,ffn\n");
                return 2;
            }
            sh.vocab = v[0]; sh.d_model = v[1]; sh.layers = v[2]; sh.q_heads = v[3]; sh.kv_heads = v[4]; sh.head_dim = v[5]; sh.ffn = v[6];
            sh.name = "custom";
        } else if (a == "--rope-theta") sh.theta = strtof(next(), nullptr);
        else if (a == "--rms-eps") sh.eps = strtof(next(), nullptr);
        else if (a == "--qkv-bias") sh.bias = true;
        else { fprintf(stderr, "Error: unknown argument '%s'\n", a.c_str()); return 2; }
    }
    if (!weights_path && !synthetic) { fprintf(stderr, "Error: give --weights FILE.safetensors or --synthetic SEED\n"); return 2; }
    if (prompt.empty() || steps == 0) { fprintf(stderr, "Error: empty prompt or zero steps\n"); return 2; }

    // ---- the file ------------------------------------------------------------------------------------------
    std::map<std::string, TensorInfo> tensors;
    std::map<std::string, GgufTensor> gguf;
    bool is_gguf = false;
    const unsigned char* file = nullptr;
    const unsigned char* data = nullptr;
    size_t file_bytes = 0;
    if (weights_path) {
        const int fd = open(weights_path, O_RDONLY);
        struct stat st;
        if (fd < 0 || fstat(fd, &st) != 0 || st.st_size < 8) { fprintf(stderr, "Error: failed to open safetensors file '%s'\n", weights_path); return 1; }
        file_bytes = (size_t)st.st_size;
        file = (const unsigned char*)mmap(nullptr, file_bytes, PROT_READ, MAP_PRIVATE, fd, 0);
        close(fd);
        if (file == MAP_FAILED) { fprintf(stderr, "Error: mmap of '%s' failed\n", weights_path); return 1; }
        if (memcmp(file, "GGUF", 4) == 0) {
            is_gguf = true;
            size_t data_start = 0;
            if (!parse_gguf(file, file_bytes, &gguf, &data_start)) { fprintf(stderr, "Error: '%s' is not a GGUF file this runner can read\n", weights_path); return 1; }
            data = file + data_start;
        } else {
            uint64_t hlen = 0;
            memcpy(&hlen, file, 8);
            if (hlen > file_bytes - 8 || !parse_header((const char*)file + 8, hlen, &tensors)) {
                fprintf(stderr, "Error: '%s' is not a safetensors file this runner can read\n", weights_path);
                return 1;
            }
            data = file + 8 + hlen;
            for (const auto& kv : tensors)
                if (kv.second.end > file_bytes - 8 - hlen || kv.second.begin > kv.second.end) { fprintf(stderr, "Error: tensor '%s' lies outside the file\n", kv.first.c_str()); return 1; }
        }
    }
    const bool tied = !weights_path ? true : (is_gguf ? gguf.find("output.weight") == gguf.end() : tensors.find("lm_head.weight") == tensors.end());

    // ---- the engine ----------------------------------------------------------------------------------------
    vb_model_desc d;
    memset(&d, 0, sizeof(d));
    d.struct_bytes = sizeof(d);
    d.vocab = sh.vocab; d.d_model = sh.d_model; d.n_layers = sh.layers; d.n_q_heads = sh.q_heads; d.n_kv_heads = sh.kv_heads;
    d.head_dim = sh.head_dim; d.ffn_dim = sh.ffn;
    d.max_seq_len = (uint32_t)(prompt.size() + steps + 1 + (speculative ? 8 : 0)); d.max_batch = 1;
    if (context_len > d.max_seq_len) d.max_seq_len = (uint32_t)context_len;  // the KV pool still holds only what is reserved below
    d.rms_eps = sh.eps; d.rope_theta = sh.theta;
    d.weight_fmt = weight_fmt;
    // embedding table and head: 16-bit when the linear layers are reduced precision (the reference's q4 table is its
    // own group-64 format), fp32 otherwise
    d.embed_fmt = weight_fmt == VB_FMT_F32 ? VB_FMT_F32 : (weight_fmt == VB_FMT_Q4G64REF ? VB_FMT_Q4G64REF : VB_FMT_F16);
    d.head_fmt = tied ? d.embed_fmt : weight_fmt;
    d.kv_blocks_total = (uint32_t)((prompt.size() + steps + 1 + (speculative ? 8 : 0) + 15) / 16);
    d.qkv_bias = sh.bias; d.tied_lm_head = tied; d.kv_block_tokens = 16; d.attn_kind = VB_ATTN_GQA; d.tp_rank = 0; d.tp_size = 1;
    vb_ctx* ctx = nullptr;
    if (vb_create(&d, 0, &ctx) != VB_OK) return fail("vb_create");

    const double t_load0 = now_ms();
    const uint32_t qdim = sh.q_heads * sh.head_dim, kvdim = sh.kv_heads * sh.head_dim;
    struct Want { int role; int layer; std::string name; uint64_t rows, cols; float mean; std::string gguf_name; };
    std::vector<Want> wants;
    wants.push_back({VB_ROLE_EMBED, 0, "model.embed_tokens.weight", sh.vocab, sh.d_model, 0.f, "token_embd.weight"});
    for (uint32_t l = 0; l < sh.layers; ++l) {
        const std::string p = "model.layers." + std::to_string(l) + ".";
        const std::string g = "blk." + std::to_string(l) + ".";  // llama.cpp names (velox_cuda_runner_k2.cu:1925-1958)
        wants.push_back({VB_ROLE_ATTN_NORM, (int)l, p + "input_layernorm.weight", 1, sh.d_model, 1.f, g + "attn_norm.weight"});
        wants.push_back({VB_ROLE_WQ, (int)l, p + "self_attn.q_proj.weight", qdim, sh.d_model, 0.f, g + "attn_q.weight"});
        wants.push_back({VB_ROLE_WK, (int)l, p + "self_attn.k_proj.weight", kvdim, sh.d_model, 0.f, g + "attn_k.weight"});
        wants.push_back({VB_ROLE_WV, (int)l, p + "self_attn.v_proj.weight", kvdim, sh.d_model, 0.f, g + "attn_v.weight"});
        if (sh.bias) {
            wants.push_back({VB_ROLE_BQ, (int)l, p + "self_attn.q_proj.bias", 1, qdim, 0.f, g + "attn_q.bias"});
            wants.push_back({VB_ROLE_BK, (int)l, p + "self_attn.k_proj.bias", 1, kvdim, 0.f, g + "attn_k.bias"});
            wants.push_back({VB_ROLE_BV, (int)l, p + "self_attn.v_proj.bias", 1, kvdim, 0.f, g + "attn_v.bias"});
        }
        wants.push_back({VB_ROLE_WO, (int)l, p + "self_attn.o_proj.weight", sh.d_model, qdim, 0.f, g + "attn_output.weight"});
        wants.push_back({VB_ROLE_MLP_NORM, (int)l, p + "post_attention_layernorm.weight", 1, sh.d_model, 1.f, g + "ffn_norm.weight"});
        wants.push_back({VB_ROLE_WGATE, (int)l, p + "mlp.gate_proj.weight", sh.ffn, sh.d_model, 0.f, g + "ffn_gate.weight"});
        wants.push_back({VB_ROLE_WUP, (int)l, p + "mlp.up_proj.weight", sh.ffn, sh.d_model, 0.f, g + "ffn_up.weight"});
        wants.push_back({VB_ROLE_WDOWN, (int)l, p + "mlp.down_proj.weight", sh.d_model, sh.ffn, 0.f, g + "ffn_down.weight"});
    }
    wants.push_back({VB_ROLE_FINAL_NORM, 0, "model.norm.weight", 1, sh.d_model, 1.f, "output_norm.weight"});
    if (!tied) wants.push_back({VB_ROLE_LM_HEAD, 0, "lm_head.weight", sh.vocab, sh.d_model, 0.f, "output.weight"});
    for (const Want& w : wants) {
        if (synthetic) {
            // stream ids as in velox_b200/modelspec.py: role * 4096 + layer
            if (vb_load_tensor_synthetic(ctx, w.role, w.layer, seed, (uint64_t)w.role * 4096 + (uint64_t)w.layer, w.mean, 0.02f, w.rows, w.cols) != VB_OK)
                return fail(w.name.c_str());
            continue;
        }
        if (is_gguf) {
            const auto gi = gguf.find(w.gguf_name);
            if (gi == gguf.end()) { fprintf(stderr, "Error: missing %s in GGUF\n", w.gguf_name.c_str()); return 1; }
            const GgufTensor& t = gi->second;
            uint64_t n = 1;
            for (uint64_t v : t.dims) n *= v;
            // GGUF lists the innermost dimension first: a matrix is {cols, rows}
            if (t.bytes == 0 || n != w.rows * w.cols || (t.dims.size() >= 2 && t.dims[0] != w.cols)) {
                fprintf(stderr, "Error: %s has an unsupported type (%u) or an unexpected shape\n", w.gguf_name.c_str(), t.type);
                return 1;
            }
            if (vb_load_tensor_gguf(ctx, w.role, w.layer, data + t.offset, (int32_t)t.type, w.rows, w.cols) != VB_OK) return fail(w.gguf_name.c_str());
            continue;
        }
        const auto it = tensors.find(w.name);
        if (it == tensors.end()) { fprintf(stderr, "Error: missing %s in safetensors\n", w.name.c_str()); return 1; }
        const TensorInfo& t = it->second;
        uint64_t n = 1;
        for (uint64_t s : t.shape) n *= s;
        const uint64_t es = t.fmt == VB_FMT_F32 ? 4 : 2;
        if (t.fmt < 0 || n != w.rows * w.cols || t.end - t.begin != n * es) {
            fprintf(stderr, "Error: %s has an unexpected dtype or shape\n", w.name.c_str());
            return 1;
        }
        if (vb_load_tensor(ctx, w.role, w.layer, data + t.begin, t.fmt, VB_LOC_HOST, w.rows, w.cols) != VB_OK) return fail(w.name.c_str());
    }
    const double load_ms = now_ms() - t_load0;
    uint64_t arena_bytes = 0;
    vb_weight_bytes(ctx, &arena_bytes);

    // ---- generation ----------------------------------------------------------------------------------------
    if (vb_seq_reserve(ctx, 0, (uint32_t)(prompt.size() + steps + (speculative ? draft_len : 0))) != VB_OK) return fail("vb_seq_reserve");
    if (temperature > 1e-5f && top_p > 0.0f) {
        if (speculative) { fprintf(stderr, "Error: speculative decoding verifies greedy tokens; drop --temperature/--top-p\n"); return 2; }
        if (vb_set_sampling(ctx, temperature, top_p, sample_seed, 0) != VB_OK) return fail("vb_set_sampling");
    }
    std::vector<uint32_t> gen(steps);
    double ttft_ms = 0.0;
    float decode_ms = 0.0f;
    vb_spec_stats spec;
    memset(&spec, 0, sizeof(spec));
    if (speculative) {
        // prefill + speculative loop in one call; the prefill is timed by a run of its own first (same prompt, same slot)
        const double t0 = now_ms();
        if (vb_prefill(ctx, 0, prompt.data(), (uint32_t)prompt.size()) != VB_OK) return fail("vb_prefill");
        if (vb_sync(ctx) != VB_OK) return fail("vb_sync");
        ttft_ms = now_ms() - t0;
        if (use_graph && vb_decode_graph_build(ctx) != VB_OK) use_graph = false;  // plain steps of the loop replay it
        const double t1 = now_ms();
        if (vb_generate_speculative(ctx, 0, prompt.data(), (uint32_t)prompt.size(), (uint32_t)steps, (uint32_t)draft_len, spec_ema, gen.data(), &spec) != VB_OK)
            return fail("vb_generate_speculative");
        decode_ms = (float)(now_ms() - t1 - ttft_ms);  // the call prefills again: count the decode part
        if (decode_ms <= 0.0f) decode_ms = (float)(now_ms() - t1);
    } else {
        const double t0 = now_ms();
        if (vb_prefill(ctx, 0, prompt.data(), (uint32_t)prompt.size()) != VB_OK) return fail("vb_prefill");
        if (vb_sync(ctx) != VB_OK) return fail("vb_sync");
        ttft_ms = now_ms() - t0;
        if (steps > 1) {
            if (use_graph && vb_decode_graph_build(ctx) != VB_OK) {
                fprintf(stderr, "Warning: CUDA Graph capture failed (%s), falling back to eager stream\n", vb_last_error());
                use_graph = false;
            }
            if (vb_decode_run(ctx, (uint32_t)(steps - 1), &decode_ms) != VB_OK) return fail("vb_decode_run");
        }
        if (vb_read_tokens(ctx, 0, (uint32_t)(prompt.size() - 1), (uint32_t)steps, gen.data()) != VB_OK) return fail("vb_read_tokens");
    }
    if (verbose)
        for (size_t s = 0; s < steps; ++s) printf("[Step %zu] Token: %u\n", s, gen[s]);
    std::vector<float> logits(sh.vocab);
    if (vb_read_logits(ctx, 0, logits.data(), logits.size()) != VB_OK) return fail("vb_read_logits");

    // ---- report (line formats of the reference runner, velox_cuda_runner.cu:589-635) ---------------------------
    printf("================================================================================\n");
    printf("VELOX B200 LIBRARY RUNTIME EXECUTION REPORT\n");
    printf("================================================================================\n");
    printf("Model                  : %s\n", sh.name);
    printf("Weights                : %s\n", synthetic ? "synthetic (counter-based generator)" : weights_path);
    printf("Weight Stream to VRAM  : %.2f ms\n", load_ms);
    printf("Weight Arena           : %.2f MiB\n", (double)arena_bytes / (1024.0 * 1024.0));
    printf("Prompt Tokens (%zu)      : [", prompt.size());
    for (size_t i = 0; i < prompt.size(); ++i) printf("%u%s", prompt[i], (i + 1 < prompt.size()) ? ", " : "");
    printf("]\n");
    printf("Generated Tokens (%zu)   : [", steps);
    for (size_t i = 0; i < steps; ++i) printf("%u%s", gen[i], (i + 1 < steps) ? ", " : "");
    printf("]\n");
    printf("TTFT (Prefill Latency) : %.3f ms\n", ttft_ms);
    if (steps > 1)
        printf("Decode Latency (%zu tok): %.3f ms (%.2f tok/s, %.3f ms/tok)\n", steps - 1, decode_ms,
               1000.0 * (double)(steps - 1) / (double)decode_ms, (double)decode_ms / (double)(steps - 1));
    printf("CUDA Graph Replay      : %s\n", use_graph ? "yes" : "no (eager launches)");
    if (speculative) {  // line formats of velox_cuda_runner_k2.cu:2417-2427
        printf("Decoding Mode          : Speculative Decoding (Prompt-Lookup, max draft K=%d)\n", draft_len);
        printf("Adaptive Policy        : EMA floor %.2f, final EMA %.2f, ladder x%u; policy-plain steps: %llu\n", spec_ema, spec.ema_final,
               spec.ladder_final, (unsigned long long)spec.plain_steps);
        printf("Draft Acceptance Rate  : %.1f%% (%llu / %llu draft tokens accepted)\n",
               spec.drafted > 0 ? 100.0 * (double)spec.accepted / (double)spec.drafted : 0.0, (unsigned long long)spec.accepted,
               (unsigned long long)spec.drafted);
        printf("Speculative Steps      : %llu forward passes for %zu generated tokens (%.2fx compression)\n", (unsigned long long)spec.steps,
               steps - 1, spec.steps > 0 ? (double)(steps - 1) / (double)spec.steps : 1.0);
    } else if (temperature > 1e-5f && top_p > 0.0f) {
        printf("Decoding Mode          : Nucleus Sampling (temperature %.3f, top-p %.3f, seed %llu)\n", temperature, top_p, (unsigned long long)sample_seed);
    } else {
        printf("Decoding Mode          : Autoregressive Standard (Single Token)\n");
    }
    std::vector<uint32_t> order(sh.vocab);
    for (uint32_t i = 0; i < sh.vocab; ++i) order[i] = i;
    const size_t k = std::min<size_t>(5, order.size());
    std::partial_sort(order.begin(), order.begin() + k, order.end(), [&](uint32_t x, uint32_t y) {
        return logits[x] > logits[y] || (logits[x] == logits[y] && x < y);
    });
    printf("Final Step Top-5 Logits:\n");
    for (size_t i = 0; i < k; ++i) printf("  #%zu: token_id=%u logit=%.6f\n", i + 1, order[i], logits[order[i]]);
    // The reference runner compares against the golden continuation of its own checkpoint and prompt
    // (velox_cuda_runner.cu:653-690); for any other weights or prompt it prints these two lines as skipped.
    printf("Parity 4-token check   : SKIPPED (Custom prompt or steps < 4)\n");
    printf("Parity 32-token check  : SKIPPED (Custom prompt or steps < 32)\n");
    printf("================================================================================\n");
    vb_destroy(ctx);
    if (file) munmap((void*)file, file_bytes);
    return 0;
}
