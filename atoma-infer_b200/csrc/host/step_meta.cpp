// The step's metadata, built on the host in two calls (so that a step costs a fixed number of calls into this
// library, whatever its size): step_begin admits and checks the entries and claims their pages; step_fill writes the
// one int32 buffer that the kernels read (header, tokens, positions, entry of each token, row starts, context
// lengths, state slots, wanted rows, block tables per cache group).  The reference builds about ten small tensors
// per step from its sequence metadata (backends/vllm/src/worker.rs:224-460).
//
// The buffer's layout is the caller's (offsets are passed in): this file only fills it.
#include <algorithm>
#include <cstdint>
#include <cstring>

#include "cache_manager.hpp"

using engine::CacheManager;

extern "C" {

// Error codes beyond CacheStatus: what was wrong with an entry; `bad_entry` names it.
enum StepStatus : int { kStepNoTokens = -20, kStepTwice = -21, kStepBadWant = -22, kStepBadToken = -23 };

// The n entries: request ids, how many tokens each brings (the tokens one after the other in `tokens`) and how many
// places of it are wanted (one after the other in `wants`).  Claims a state slot for requests seen for the first time
// and the pages all tokens need.  Outputs per entry: tokens already cached, state slot, whether the request starts
// (nothing cached yet); per cache group: the longest block table among the entries.  On an error nothing of the
// failing entry stays (a request that this call added is freed again); entries before it keep their pages, as they
// would after a step that ran.  vocab: token ids must lie in [0, vocab), except the one negative id -1 - slot that a
// single decode token of a request with cached tokens may bring ("the token the sampler left on the device for my
// slot").
int cm_step_begin(void* h, int n, const int64_t* reqs, const int32_t* ntok, const int32_t* tokens, const int32_t* want_count,
                  const int32_t* wants, int vocab, int64_t* ctx_out, int32_t* slot_out, int32_t* new_out,
                  int32_t* table_len_out, int32_t* bad_entry) {
    auto* cm = static_cast<CacheManager*>(h);
    const int groups = cm->num_groups();
    for (int g = 0; g < groups; ++g) table_len_out[g] = 1;
    int64_t t0 = 0, w0 = 0;
    for (int k = 0; k < n; ++k) {
        *bad_entry = k;
        if (ntok[k] <= 0) return kStepNoTokens;
        for (int j = 0; j < k; ++j)
            if (reqs[j] == reqs[k]) return kStepTwice;
        const bool added = !cm->has_request(reqs[k]);
        const int slot = added ? cm->add_request(reqs[k]) : cm->state_slot(reqs[k]);
        if (slot < 0) return slot;
        const int64_t ctx = cm->num_tokens(reqs[k]);
        int err = engine::kOk;
        for (int j = 0; j < want_count[k]; ++j)
            if (wants[w0 + j] < 0 || wants[w0 + j] >= ntok[k]) err = kStepBadWant;
        const int32_t lo = *std::min_element(tokens + t0, tokens + t0 + ntok[k]);
        const int32_t hi = *std::max_element(tokens + t0, tokens + t0 + ntok[k]);
        if (err == engine::kOk && (hi >= vocab || (lo < 0 && !(ntok[k] == 1 && ctx > 0 && lo == -1 - slot)))) err = kStepBadToken;
        if (err == engine::kOk) err = cm->reserve(reqs[k], ctx + ntok[k]);
        if (err != engine::kOk) {
            if (added) cm->free_request(reqs[k]);
            return err;
        }
        ctx_out[k] = ctx;
        slot_out[k] = slot;
        new_out[k] = ctx == 0;
        for (int g = 0; g < groups; ++g) table_len_out[g] = std::max(table_len_out[g], cm->table_len(reqs[k], g));
        t0 += ntok[k];
        w0 += want_count[k];
    }
    *bad_entry = -1;
    return engine::kOk;
}

// Fills the buffer.  T, S, R: tokens, entries and wanted rows of the step; cap_T, cap_S, cap_R: what the arrays are
// laid out for (a captured graph's fixed sizes; the header holds the true counts).  Offsets in ints: tokens,
// positions, token_entry, cu, ctx, slots, rows, then per group its tables' offset and row stride.  tokens: the
// entries' tokens one after the other; wants: their wanted places likewise, want_count per entry.
void cm_step_fill(void* h, int n, const int64_t* reqs, const int32_t* ntok, const int64_t* ctx, const int32_t* slots,
                  const int32_t* tokens, const int32_t* want_count, const int32_t* wants, int32_t* buf, int header_ints,
                  int cap_T, int cap_S, int cap_R, int off_tokens, int off_positions, int off_entry, int off_cu, int off_ctx,
                  int off_slots, int off_rows, const int32_t* table_off, const int32_t* table_stride, int meta_num_tokens,
                  int meta_num_entries, int meta_num_rows, int meta_bt_stride, int meta_bt_offset) {
    auto* cm = static_cast<CacheManager*>(h);
    const int groups = cm->num_groups();
    std::memset(buf, 0, sizeof(int32_t) * (size_t)header_ints);
    int T = 0, R = 0;
    for (int k = 0; k < n; ++k) {
        const int a = T;
        for (int i = 0; i < ntok[k]; ++i) {
            buf[off_tokens + a + i] = tokens[a + i];
            buf[off_positions + a + i] = (int32_t)(ctx[k] + i);
            buf[off_entry + a + i] = k;
        }
        buf[off_cu + k] = a;
        buf[off_ctx + k] = (int32_t)ctx[k];
        buf[off_slots + k] = slots[k];
        for (int j = 0; j < want_count[k]; ++j) buf[off_rows + R + j] = a + wants[R + j];
        R += want_count[k];
        T += ntok[k];
    }
    buf[meta_num_tokens] = T;
    buf[meta_num_entries] = n;
    buf[meta_num_rows] = R;
    // padding of a captured graph's arrays: harmless values (token 0, position 0, entry 0, rows of length 0)
    for (int k = n; k <= cap_S; ++k) buf[off_cu + k] = T;
    for (int i = T; i < cap_T; ++i) buf[off_tokens + i] = buf[off_positions + i] = buf[off_entry + i] = 0;
    for (int k = n; k < cap_S; ++k) buf[off_ctx + k] = buf[off_slots + k] = 0;
    for (int j = R; j < std::max(cap_R, 1); ++j) buf[off_rows + j] = 0;
    for (int g = 0; g < groups; ++g) {
        buf[meta_bt_stride + g] = table_stride[g];
        buf[meta_bt_offset + g] = table_off[g];
        int32_t* tab = buf + table_off[g];
        std::fill(tab, tab + (size_t)cap_S * table_stride[g], -1);
        for (int k = 0; k < n; ++k) cm->table(reqs[k], g, tab + (size_t)k * table_stride[g], table_stride[g]);
    }
}

}  // extern "C"
