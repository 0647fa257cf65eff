// The layout of one step in the pinned host buffer: what the step function uploads before it launches.
//
// A step is a list of (request, its next tokens, the places among them whose logits are wanted).  The
// reference rebuilds per-token positions and per-sequence slot lists on the host every step
// (src/batch.rs:10-83) and uploads them; here the same work fills fixed sections of one pinned buffer:
// token ids, positions, the sequence of every token, per sequence its state slot, first token and new
// length, the wanted rows, and the block-table entries the device does not have yet.  Sequences that
// bring exactly one token come first (the decode kernels take the leading one-token sequences).
#pragma once
#include <cstdint>

#include "cache_manager.h"

namespace carbon {

enum LayoutStatus {
    LAYOUT_OK = 0,
    LAYOUT_NO_ENTRIES = -101,
    LAYOUT_TOO_MANY_ENTRIES = -102,
    LAYOUT_TOO_MANY_TOKENS = -103,
    LAYOUT_TOO_MANY_WANTS = -104,     // more wanted places than tokens: a place is named twice
    LAYOUT_EMPTY_ENTRY = -105,        // detail[0]: the request
    LAYOUT_TWICE = -106,              // detail[0]: the request that appears twice
    LAYOUT_BAD_WANT = -107,           // detail[0]: the request, detail[1]: the place, detail[2]: its tokens
    // a CacheStatus (> -100) from reserving pages: detail[0]: the request, detail[1]: the length asked for
};

struct StepLayoutArgs {
    // the step, entry after entry
    int n;
    const int64_t* ids;
    const int32_t* counts;            // tokens of each entry
    const int32_t* tokens;            // all tokens, entry after entry
    const int32_t* want_counts;       // wanted places of each entry
    const int32_t* wants;             // all wanted places (indices into the entry's own tokens)
    int max_step_tokens;
    // sections of the pinned buffer
    int32_t* tok;
    int32_t* pos;
    int32_t* seq_of_token;
    int32_t* seq_slot;
    int32_t* q_start;                 // n + 1
    int32_t* ctx_len;
    int32_t* rows;
    // block-table entries the device lacks: synced[g * max_requests + slot] entries of a row are there already;
    // new ones are appended to upd_idx / upd_val of the group (upd_stride entries apart), counted in n_upd[g]
    int64_t* synced;
    int32_t* upd_idx;
    int32_t* upd_val;
    int upd_stride;
    int32_t* n_upd;
    // results, per sequence in the step's order (one-token sequences first)
    int64_t* out_ids;
    int32_t* out_slot;
    int32_t* out_ctx_before;
    int32_t* out_new_len;
    int32_t* out;                     // T, wanted rows, leading one-token sequences, largest position, longest context
    int64_t* detail;                  // 3 values describing an error
};

// Checks the step, reserves its pages and fills the sections.  On an error nothing is changed but pages
// that entries before the faulty one have reserved (they stay with their requests).
int layout_step(CacheManager& cm, const StepLayoutArgs& a);

}  // namespace carbon
