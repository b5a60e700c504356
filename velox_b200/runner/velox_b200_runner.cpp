// Stand-alone runner over the C ABI of libvelox_b200: the role of the reference's host runner
// (src/runners/velox_cuda_runner.cu:327-700) with its command line and report lines, for any Llama-style
// decoder shape instead of one compiled-in model.
//
//   velox_b200_runner --weights model.safetensors --tokens 1,2,3 --steps 32 [--quantize f16|q4_0|q4g32|i8]
//                     [--model smollm-135m | --dims vocab,d_model,layers,q_heads,kv_heads,head_dim,ffn]
//                     [--rope-theta T] [--rms-eps E] [--qkv-bias] [--synthetic SEED] [--no-cuda-graph] [--verbose]
//
// Weights come from a safetensors file (F32 / F16 / BF16 tensors under the Hugging Face Llama names listed in
// src/runtime.rs:1274-1290; a missing lm_head.weight means tied embeddings) or, with --synthetic, from the
// library's counter-based generator.  Everything numerical happens in the library; this file is host plumbing.
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
    const bool tied = weights_path ? tensors.find("lm_head.weight") == tensors.end() : true;

    // ---- the engine ----------------------------------------------------------------------------------------
    vb_model_desc d;
    memset(&d, 0, sizeof(d));
    d.struct_bytes = sizeof(d);
    d.vocab = sh.vocab; d.d_model = sh.d_model; d.n_layers = sh.layers; d.n_q_heads = sh.q_heads; d.n_kv_heads = sh.kv_heads;
    d.head_dim = sh.head_dim; d.ffn_dim = sh.ffn;
    d.max_seq_len = (uint32_t)(prompt.size() + steps + 1); d.max_batch = 1;
    d.rms_eps = sh.eps; d.rope_theta = sh.theta;
    d.weight_fmt = weight_fmt;
    // embedding table and head: 16-bit when the linear layers are reduced precision (the reference's q4 table is its
    // own group-64 format), fp32 otherwise
    d.embed_fmt = weight_fmt == VB_FMT_F32 ? VB_FMT_F32 : (weight_fmt == VB_FMT_Q4G64REF ? VB_FMT_Q4G64REF : VB_FMT_F16);
    d.head_fmt = tied ? d.embed_fmt : weight_fmt;
    d.qkv_bias = sh.bias; d.tied_lm_head = tied; d.kv_block_tokens = 16; d.attn_kind = VB_ATTN_GQA; d.tp_rank = 0; d.tp_size = 1;
    vb_ctx* ctx = nullptr;
    if (vb_create(&d, 0, &ctx) != VB_OK) return fail("vb_create");

    const double t_load0 = now_ms();
    const uint32_t qdim = sh.q_heads * sh.head_dim, kvdim = sh.kv_heads * sh.head_dim;
    struct Want { int role; int layer; std::string name; uint64_t rows, cols; float mean; };
    std::vector<Want> wants;
    wants.push_back({VB_ROLE_EMBED, 0, "model.embed_tokens.weight", sh.vocab, sh.d_model, 0.f});
    for (uint32_t l = 0; l < sh.layers; ++l) {
        const std::string p = "model.layers." + std::to_string(l) + ".";
        wants.push_back({VB_ROLE_ATTN_NORM, (int)l, p + "input_layernorm.weight", 1, sh.d_model, 1.f});
        wants.push_back({VB_ROLE_WQ, (int)l, p + "self_attn.q_proj.weight", qdim, sh.d_model, 0.f});
        wants.push_back({VB_ROLE_WK, (int)l, p + "self_attn.k_proj.weight", kvdim, sh.d_model, 0.f});
        wants.push_back({VB_ROLE_WV, (int)l, p + "self_attn.v_proj.weight", kvdim, sh.d_model, 0.f});
        if (sh.bias) {
            wants.push_back({VB_ROLE_BQ, (int)l, p + "self_attn.q_proj.bias", 1, qdim, 0.f});
            wants.push_back({VB_ROLE_BK, (int)l, p + "self_attn.k_proj.bias", 1, kvdim, 0.f});
            wants.push_back({VB_ROLE_BV, (int)l, p + "self_attn.v_proj.bias", 1, kvdim, 0.f});
        }
        wants.push_back({VB_ROLE_WO, (int)l, p + "self_attn.o_proj.weight", sh.d_model, qdim, 0.f});
        wants.push_back({VB_ROLE_MLP_NORM, (int)l, p + "post_attention_layernorm.weight", 1, sh.d_model, 1.f});
        wants.push_back({VB_ROLE_WGATE, (int)l, p + "mlp.gate_proj.weight", sh.ffn, sh.d_model, 0.f});
        wants.push_back({VB_ROLE_WUP, (int)l, p + "mlp.up_proj.weight", sh.ffn, sh.d_model, 0.f});
        wants.push_back({VB_ROLE_WDOWN, (int)l, p + "mlp.down_proj.weight", sh.d_model, sh.ffn, 0.f});
    }
    wants.push_back({VB_ROLE_FINAL_NORM, 0, "model.norm.weight", 1, sh.d_model, 1.f});
    if (!tied) wants.push_back({VB_ROLE_LM_HEAD, 0, "lm_head.weight", sh.vocab, sh.d_model, 0.f});
    for (const Want& w : wants) {
        if (synthetic) {
            // stream ids as in velox_b200/modelspec.py: role * 4096 + layer
            if (vb_load_tensor_synthetic(ctx, w.role, w.layer, seed, (uint64_t)w.role * 4096 + (uint64_t)w.layer, w.mean, 0.02f, w.rows, w.cols) != VB_OK)
                return fail(w.name.c_str());
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
    if (vb_seq_reserve(ctx, 0, (uint32_t)(prompt.size() + steps)) != VB_OK) return fail("vb_seq_reserve");
    const double t0 = now_ms();
    if (vb_prefill(ctx, 0, prompt.data(), (uint32_t)prompt.size()) != VB_OK) return fail("vb_prefill");
    if (vb_sync(ctx) != VB_OK) return fail("vb_sync");
    const double ttft_ms = now_ms() - t0;
    float decode_ms = 0.0f;
    if (steps > 1) {
        if (use_graph && vb_decode_graph_build(ctx) != VB_OK) {
            fprintf(stderr, "Warning: CUDA Graph capture failed (%s), falling back to eager stream\n", vb_last_error());
            use_graph = false;
        }
        if (vb_decode_run(ctx, (uint32_t)(steps - 1), &decode_ms) != VB_OK) return fail("vb_decode_run");
    }
    std::vector<uint32_t> gen(steps);
    if (vb_read_tokens(ctx, 0, (uint32_t)(prompt.size() - 1), (uint32_t)steps, gen.data()) != VB_OK) return fail("vb_read_tokens");
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
    std::vector<uint32_t> order(sh.vocab);
    for (uint32_t i = 0; i < sh.vocab; ++i) order[i] = i;
    const size_t k = std::min<size_t>(5, order.size());
    std::partial_sort(order.begin(), order.begin() + k, order.end(), [&](uint32_t x, uint32_t y) {
        return logits[x] > logits[y] || (logits[x] == logits[y] && x < y);
    });
    printf("Final Step Top-5 Logits:\n");
    for (size_t i = 0; i < k; ++i) printf("  #%zu: token_id=%u logit=%.6f\n", i + 1, order[i], logits[order[i]]);
    printf("================================================================================\n");
    vb_destroy(ctx);
    if (file) munmap((void*)file, file_bytes);
    return 0;
}
