#include "step_layout.h"

#include <algorithm>
#include <utility>
#include <vector>

namespace carbon {

int layout_step(CacheManager& cm, const StepLayoutArgs& a) {
    const int n = a.n;
    if (n <= 0) return LAYOUT_NO_ENTRIES;
    if (n > cm.max_requests()) {
        a.detail[0] = n;
        a.detail[1] = cm.max_requests();
        return LAYOUT_TOO_MANY_ENTRIES;
    }
    long long T = 0, W = 0;
    for (int i = 0; i < n; ++i) {
        if (a.counts[i] <= 0) {
            a.detail[0] = a.ids[i];
            return LAYOUT_EMPTY_ENTRY;
        }
        T += a.counts[i];
        W += a.want_counts[i];
    }
    if (T > a.max_step_tokens) {
        a.detail[0] = T;
        a.detail[1] = a.max_step_tokens;
        return LAYOUT_TOO_MANY_TOKENS;
    }
    if (W > T) return LAYOUT_TOO_MANY_WANTS;
    {
        std::vector<int64_t> sorted(a.ids, a.ids + n);
        std::sort(sorted.begin(), sorted.end());
        for (int i = 1; i < n; ++i)
            if (sorted[i] == sorted[i - 1]) {
                a.detail[0] = sorted[i];
                return LAYOUT_TWICE;
            }
        long long w0 = 0;
        for (int i = 0; i < n; ++i) {
            for (int k = 0; k < a.want_counts[i]; ++k) {
                int w = a.wants[w0 + k];
                if (w < 0 || w >= a.counts[i]) {
                    a.detail[0] = a.ids[i];
                    a.detail[1] = w;
                    a.detail[2] = a.counts[i];
                    return LAYOUT_BAD_WANT;
                }
            }
            w0 += a.want_counts[i];
        }
        for (int i = 0; i < n; ++i)
            if (cm.slot_of(a.ids[i]) < 0) {
                a.detail[0] = a.ids[i];
                a.detail[1] = 0;
                return CACHE_UNKNOWN;
            }
    }
    // one-token sequences first, each kind in the order given
    std::vector<int> order;
    order.reserve(n);
    for (int i = 0; i < n; ++i)
        if (a.counts[i] == 1) order.push_back(i);
    for (int i = 0; i < n; ++i)
        if (a.counts[i] != 1) order.push_back(i);
    std::vector<long long> token_start(n), want_start(n);
    {
        long long t = 0, w = 0;
        for (int i = 0; i < n; ++i) {
            token_start[i] = t;
            want_start[i] = w;
            t += a.counts[i];
            w += a.want_counts[i];
        }
    }
    const int groups = cm.num_groups(), max_req = cm.max_requests(), max_pages = cm.max_pages_per_request();
    std::vector<std::pair<size_t, int64_t>> touched;      // entries of `synced` to put back if a later entry fails
    for (int g = 0; g < groups; ++g) a.n_upd[g] = 0;
    std::vector<int> start_of(n);
    int off = 0, n_decode = 0, max_position = 0, max_ctx = 0;
    for (int bi = 0; bi < n; ++bi) {
        const int i = order[bi];
        const int64_t id = a.ids[i];
        const int cnt = a.counts[i];
        const int start = cm.length_of(id), slot = cm.slot_of(id);
        const int rc = cm.reserve(id, start + cnt);
        if (rc != CACHE_OK) {
            for (auto it = touched.rbegin(); it != touched.rend(); ++it) a.synced[it->first] = it->second;
            a.detail[0] = id;
            a.detail[1] = start + cnt;
            return rc;
        }
        const int32_t* toks = a.tokens + token_start[i];
        for (int k = 0; k < cnt; ++k) {
            a.tok[off + k] = toks[k];
            a.pos[off + k] = start + k;
            a.seq_of_token[off + k] = bi;
        }
        a.seq_slot[bi] = slot;
        a.q_start[bi] = off;
        a.ctx_len[bi] = start + cnt;
        start_of[i] = off;
        a.out_ids[bi] = id;
        a.out_slot[bi] = slot;
        a.out_ctx_before[bi] = start;
        a.out_new_len[bi] = start + cnt;
        if (cnt == 1 && bi == n_decode) ++n_decode;
        max_position = std::max(max_position, start + cnt - 1);
        max_ctx = std::max(max_ctx, start + cnt);
        for (int g = 0; g < groups; ++g) {
            const int ps = cm.group(g).page_size;
            const int hi = (start + cnt + ps - 1) / ps;
            const size_t at = (size_t)g * max_req + slot;
            const int lo = (int)a.synced[at];
            if (hi <= lo) continue;
            const int32_t* row = cm.table(g) + (size_t)slot * max_pages;
            int32_t* idx = a.upd_idx + (size_t)g * a.upd_stride;
            int32_t* val = a.upd_val + (size_t)g * a.upd_stride;
            for (int p = lo; p < hi && a.n_upd[g] < a.upd_stride; ++p) {
                idx[a.n_upd[g]] = slot * max_pages + p;
                val[a.n_upd[g]] = row[p];
                ++a.n_upd[g];
            }
            touched.emplace_back(at, a.synced[at]);
            a.synced[at] = hi;
        }
        off += cnt;
    }
    a.q_start[n] = off;
    int n_rows = 0;
    for (int i = 0; i < n; ++i)
        for (int k = 0; k < a.want_counts[i]; ++k) a.rows[n_rows++] = start_of[i] + a.wants[want_start[i] + k];
    a.out[0] = off;
    a.out[1] = n_rows;
    a.out[2] = n_decode;
    a.out[3] = max_position;
    a.out[4] = max_ctx;
    return LAYOUT_OK;
}

}  // namespace carbon
