// Prompt-lookup speculative decoding over the decode engine.
//
// Reference: the speculative loop of the K2 runner (src/runners/velox_cuda_runner_k2.cu:2127-2311): the host drafts
// up to K tokens by finding the most recent earlier occurrence of the history's last n-gram (:1572-1611), one
// batched forward pass verifies the K+1 candidate rows (:1539-1566, lm_head + per-row argmax :1327-1480), and the
// host keeps the drafts up to the first disagreement plus the pass's own next token (:2259-2296).  An EMA of the
// acceptance rate sizes the draft and pauses drafting when it pays too rarely (:2160-2225).
//
// Here the verify pass is one launch sequence over K+1 rows that are consecutive positions of the sequence: the
// rows share every weight pass (multi-row kernels), their K/V rows are appended before attention, row j attends
// positions 0..pos+j.  Rows after a rejected draft leave stale K/V behind; those positions are rewritten before
// anything reads them again, exactly as in the reference.
#include <math.h>
#include <string.h>

#include <vector>

#include "vb_ctx.cuh"

namespace vb {

namespace {

// rows j < n: candidate j at position first + j
__global__ void k_set_verify_state(SeqState* state, const uint32_t* tokens, uint32_t first, uint32_t n) {
    const uint32_t j = threadIdx.x;
    if (j < n) {
        state[j].token = tokens[j];
        state[j].pos = first + j;
        state[j].active = 1u;
        state[j].limit = 0;  // the host checked the rows against the reservation
    }
}
__global__ void k_fill_verify_table(int32_t* dst, const int32_t* src_row, uint32_t max_blocks) {
    for (uint32_t i = threadIdx.x; i < max_blocks; i += blockDim.x) dst[(size_t)blockIdx.x * max_blocks + i] = src_row[i];
}

// src/runners/velox_cuda_runner_k2.cu:1572-1611
int prompt_lookup_draft(const uint32_t* history, size_t history_len, uint32_t* draft, int max_draft) {
    if (history_len < 2 || max_draft <= 0) return 0;
    for (int n = 3; n >= 1; --n) {
        if (history_len < (size_t)(n + 1)) continue;
        const uint32_t* needle = history + history_len - n;
        for (long long i = (long long)(history_len - n - 1); i >= 0; --i) {
            if (memcmp(history + i, needle, (size_t)n * sizeof(uint32_t)) != 0) continue;
            const size_t start = (size_t)i + n;
            if (start >= history_len - n) continue;
            int count = (int)((history_len - n) - start);
            const int limit = (n == 1 && max_draft > 2) ? 2 : max_draft;
            if (count > limit) count = limit;
            for (int d = 0; d < count; ++d) draft[d] = history[start + d];
            return count;
        }
    }
    return 0;
}

// The adaptive draft policy, src/runners/velox_cuda_runner_k2.cu:2160-2225 and :2298-2303.
struct Policy {
    int max_draft_len;
    float floor, ema = 0.70f;
    int plain_stride = 1, plain_since_spec = 0;
    int width(int K, size_t remaining) {
        static const float thr[5] = {0.80f, 0.60f, 0.40f, 0.20f, 0.0f};
        static const float mul[5] = {1.0f, 0.75f, 0.50f, 0.25f, 0.0f};
        if ((size_t)K > remaining) K = (int)remaining;
        if (K > 0) {
            float k_mult = 0.0f;
            for (int i = 0; i < 5; ++i)
                if (ema >= thr[i]) { k_mult = mul[i]; break; }
            int k_cap = (int)((float)max_draft_len * k_mult * (0.4f + 0.6f * fminf(ema, 1.0f)));
            if (k_cap < 1) k_cap = 1;
            if (K > k_cap) K = k_cap;
            if ((size_t)K > remaining) K = (int)remaining;
        }
        bool spec;
        if (ema >= floor || K <= 0) {
            spec = K > 0;
            plain_since_spec = 0;
        } else if (plain_since_spec >= plain_stride) {
            spec = true;
            plain_since_spec = 0;
            plain_stride = plain_stride < 64 ? plain_stride * 2 : 64;
        } else {
            spec = false;
            plain_since_spec++;
        }
        return spec ? K : 0;
    }
    void update(int accepted, int K) { ema = (1.0f - 0.35f) * ema + 0.35f * ((float)accepted / (float)K); }
};

constexpr uint32_t SPEC_ROWS = 8;  // 1 + at most 7 drafts

int32_t ensure_spec_buffers(vb_ctx* c) {
    int32_t rc = ensure_chunk_buffers(c, SPEC_ROWS);
    if (rc != VB_OK) return rc;
    if (c->spec_logits) return VB_OK;
    if ((rc = dev_alloc(&c->spec_logits, (uint64_t)SPEC_ROWS * c->vocab)) != VB_OK) return rc;
    if ((rc = dev_alloc(&c->spec_cand_v, (uint64_t)SPEC_ROWS * argmax_chunks(c->vocab))) != VB_OK) return rc;
    if ((rc = dev_alloc(&c->spec_cand_i, (uint64_t)SPEC_ROWS * argmax_chunks(c->vocab))) != VB_OK) return rc;
    if ((rc = dev_alloc(&c->spec_tokens, (uint64_t)2 * SPEC_ROWS)) != VB_OK) return rc;  // candidates, then winners
    return VB_OK;
}

// One verify pass: rows = candidates at positions pos..pos+B-1 of `slot`; winners[j] = greedy token after row j.
int32_t verify_pass(vb_ctx* c, int32_t slot, const uint32_t* cand, uint32_t B, uint32_t pos, uint32_t* winners) {
    uint32_t* d_cand = c->spec_tokens;
    uint32_t* d_win = c->spec_tokens + SPEC_ROWS;
    VB_CUDA(cudaMemcpyAsync(d_cand, cand, B * 4, cudaMemcpyHostToDevice, c->stream));
    VB_CUDA(launch(lcfg(c, false), k_set_verify_state, dim3(1), dim3(32), 0, c->pfc_state, (const uint32_t*)d_cand, pos, B));
    VB_CUDA(launch(lcfg(c, false), k_fill_verify_table, dim3(B), dim3(128), 0, c->pfc_table,
                   (const int32_t*)(c->block_table_dev + (size_t)slot * c->max_blocks), c->max_blocks));
    StepIO io{c->pfc_hidden, c->pfc_qkv, c->pfc_q, c->pfc_attn, c->pfc_act, nullptr, c->pfc_table, B, false};
    VB_CUDA(enqueue_step(c, c->pfc_state, false, io));
    // final norm + lm_head for every row, then the per-row argmax (lowest index wins ties)
    GemvArgs h;
    h.state = c->pfc_state; h.batch = B; h.x = c->pfc_hidden; h.dst = c->spec_logits;
    h.norm_w = c->tensor(VB_ROLE_FINAL_NORM, 0).m.data; h.norm_fmt = c->tensor(VB_ROLE_FINAL_NORM, 0).m.fmt; h.eps = c->d.rms_eps;
    h.w = c->tensor(VB_ROLE_LM_HEAD, 0).m;
    h.max_ring = c->head_ring;
    VB_CUDA(gemv(lcfg(c, true), h, c->gemv_path));
    VB_CUDA(argmax(lcfg(c, true), d_win, c->spec_logits, c->vocab, B, c->spec_cand_v, c->spec_cand_i, nullptr, nullptr, 0));
    VB_CUDA(cudaMemcpyAsync(winners, d_win, B * 4, cudaMemcpyDeviceToHost, c->stream));
    VB_CUDA(cudaStreamSynchronize(c->stream));
    return VB_OK;
}

}  // namespace

}  // namespace vb

using namespace vb;

extern "C" int32_t vb_generate_speculative(vb_ctx* c, int32_t slot, const uint32_t* prompt, uint32_t n_prompt, uint32_t n_new,
                                           uint32_t max_draft_len, float ema_floor, uint32_t* out_tokens, vb_spec_stats* stats) {
    int32_t rc = check_ready(c, "vb_generate_speculative");
    if (rc != VB_OK) return rc;
    VB_REQUIRE(slot >= 0 && (uint32_t)slot < c->d.max_batch, "vb_generate_speculative: slot %d out of range", slot);
    VB_REQUIRE(prompt && n_prompt > 0 && out_tokens && n_new > 0, "vb_generate_speculative: empty prompt or output");
    VB_REQUIRE(max_draft_len >= 1 && max_draft_len <= 7, "vb_generate_speculative: draft length %u outside 1..7", max_draft_len);
    if (c->d.tp_size > 1) { set_error("vb_generate_speculative: the multi-row verify pass runs unsharded"); return VB_ERR_UNSUPPORTED; }
    for (uint32_t s = 0; s < c->d.max_batch; ++s)
        if ((int32_t)s != slot && c->maybe_active[s]) { set_error("vb_generate_speculative: slot %u is active; speculative decoding serves one sequence", s); return VB_ERR_STATE; }
    const uint64_t reserved = (uint64_t)c->slot_blocks[slot] * c->d.kv_block_tokens;
    // a verify pass writes K/V for up to max_draft_len rows past the last token that is kept
    VB_REQUIRE((uint64_t)n_prompt + n_new + max_draft_len <= reserved,
               "vb_generate_speculative: needs %llu reserved tokens (prompt + new + draft rows), the slot has %llu",
               (unsigned long long)n_prompt + n_new + max_draft_len, (unsigned long long)reserved);
    if (ema_floor < 0.0f) ema_floor = 0.0f;
    if (ema_floor > 0.95f) ema_floor = 0.95f;
    VB_CUDA(cudaSetDevice(c->device));
    if ((rc = ensure_spec_buffers(c)) != VB_OK) return rc;
    vb_spec_stats st;
    memset(&st, 0, sizeof(st));

    if ((rc = vb_prefill(c, slot, prompt, n_prompt)) != VB_OK) return rc;
    uint32_t next = 0;
    if ((rc = vb_read_tokens(c, slot, n_prompt - 1, 1, &next)) != VB_OK) return rc;
    std::vector<uint32_t> history(prompt, prompt + n_prompt);
    history.reserve((size_t)n_prompt + n_new + 8);
    history.push_back(next);
    out_tokens[0] = next;
    uint32_t gen = 1, pos = n_prompt;
    Policy pol;
    pol.max_draft_len = (int)max_draft_len;
    pol.floor = ema_floor;
    while (gen < n_new) {
        st.steps++;
        uint32_t draft[8];
        int K = prompt_lookup_draft(history.data(), history.size(), draft, (int)max_draft_len);
        K = pol.width(K, n_new - gen);
        if (K == 0) {
            // plain step through the decode path (graph replay when one is built)
            st.plain_steps++;
            if ((rc = vb_seq_set(c, slot, next, pos, 1)) != VB_OK) return rc;
            if ((rc = vb_decode_run(c, 1, nullptr)) != VB_OK) return rc;
            if ((rc = vb_read_tokens(c, slot, pos, 1, &next)) != VB_OK) return rc;
            pos++;
            out_tokens[gen++] = next;
            history.push_back(next);
            continue;
        }
        st.drafted += (uint64_t)K;
        const uint32_t B = (uint32_t)K + 1;
        uint32_t cand[SPEC_ROWS], winners[SPEC_ROWS];
        cand[0] = next;
        for (int i = 0; i < K; ++i) cand[i + 1] = draft[i];
        if ((rc = verify_pass(c, slot, cand, B, pos, winners)) != VB_OK) return rc;
        int accepted = 0;
        for (uint32_t t = 0; t < B && gen < n_new; ++t) {
            const uint32_t winner = winners[t];
            if (t < B - 1) {
                if (winner == cand[t + 1]) {
                    accepted++;
                    st.accepted++;
                    out_tokens[gen++] = cand[t + 1];
                    history.push_back(cand[t + 1]);
                    if (gen == n_new) { next = cand[t + 1]; pos += t + 1; }
                } else {
                    out_tokens[gen++] = winner;
                    history.push_back(winner);
                    next = winner;
                    pos += t + 1;
                    break;
                }
            } else {
                out_tokens[gen++] = winner;
                history.push_back(winner);
                next = winner;
                pos += B;
            }
        }
        pol.update(accepted, K);
    }
    st.ema_final = pol.ema;
    st.ladder_final = (uint32_t)pol.plain_stride;
    if (stats) *stats = st;
    // leave the slot where plain decoding continues: the last token still to be fed, at its position
    if ((rc = vb_seq_set(c, slot, next, pos, 1)) != VB_OK) return rc;
    return vb_sync(c);
}
