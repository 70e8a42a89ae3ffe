// Host code: fills the packed int32 buffer of a decode step (every request brings one
// token) straight into pinned memory, for the captured step's fixed layout.
//
// The reference builds its batch descriptor in native code too
// (crates/pagedllm/src/batch.rs:67-94, and the per-layer table uploads of
// crates/pagedllm/src/kernels/paged_attention.rs:114-123); here the whole step is one
// buffer, and this function is the fast path of engine/step.py's StepPacker.pack for
// the step that is replayed thousands of times: same layout, same attention work items
// (kernels/attention_plan.py, whose arithmetic is restated below and compared with it
// in the tests), a few microseconds instead of the Python's 150.
#include <stdint.h>
#include <string.h>

#include "common.cuh"

struct PllmGroupPack {
    const int* const* tables;   // [n] each request's block table of this group (int32; -1: page given back)
    const int* table_len;       // [n] entries in each
    int window;                 // 0: every key stays
    int ctas_per_item;          // CTAs the attention kernel launches per work item
    int max_work, max_red, max_parts;                                    // capacities of the captured step
    int plans;                  // 0: the group's mixers take no attention work items (the offsets of work and red are unused)
    int off_slots, off_tables, off_n_work, off_n_red, off_work, off_red; // offsets in int32 units
};

enum : int {
    PLLM_PACK_TOKEN = -10,      // a token id outside the vocabulary
    PLLM_PACK_POSITION = -11,   // a position at or past max_position_embeddings
    PLLM_PACK_NO_PAGE = -12,    // no page reserved for the token's position
    PLLM_PACK_FREED_PAGE = -13, // the token's page was given back
    PLLM_PACK_WORK = -14,       // the attention work does not fit the capacities
    PLLM_PACK_WIDTH = -15,      // a block table wider than the step's capacity
    PLLM_PACK_SIZE = -16,       // more requests than the capacities, or a buffer too short
};

static const int SPLIT_ALIGN = 64;
static const int MAX_SPLITS = 128;

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// tokens, positions, state_slots, temperature, uniform: one per request (temperature and
// uniform may be null).  out: the step's buffer (out_len int32), zeroed and filled here.
// On a refusal *err_request names the request it was about (or -1).
PLLM_EXPORT int pllm_pack_decode_step(int* out, int out_len, int n, const int* tokens, const int* positions,
                                      const int* state_slots, const float* temperature, const float* uniform,
                                      int cap_tokens, int cap_wanted, int cap_segments, int table_width, int page_size,
                                      int vocab, int max_positions, int target_ctas, int min_split_keys, int off_tokens,
                                      int off_positions, int off_rows, int off_segments, int off_temperature,
                                      int off_uniform, int n_groups, const PllmGroupPack* groups, int* err_request) {
    *err_request = -1;
    if (n <= 0 || n > cap_tokens || n > cap_wanted || n > cap_segments || page_size <= 0 || min_split_keys <= 0)
        return PLLM_PACK_SIZE;
    memset(out, 0, (size_t)out_len * sizeof(int));
    for (int i = 0; i < n; i++) {
        if (tokens[i] < 0 || tokens[i] >= vocab) { *err_request = i; return PLLM_PACK_TOKEN; }
        if (positions[i] < 0 || positions[i] >= max_positions) { *err_request = i; return PLLM_PACK_POSITION; }
        out[off_tokens + i] = tokens[i];
        out[off_positions + i] = positions[i];
        out[off_rows + i] = i;
        int* seg = out + off_segments + 4 * i;
        seg[0] = i; seg[1] = 1; seg[2] = positions[i]; seg[3] = state_slots[i];
        if (temperature) memcpy(out + off_temperature + i, temperature + i, sizeof(float));
        if (uniform) memcpy(out + off_uniform + i, uniform + i, sizeof(float));
    }
    for (int gi = 0; gi < n_groups; gi++) {
        const PllmGroupPack& g = groups[gi];
        int* slots = out + g.off_slots;
        int* tables = out + g.off_tables;
        for (int i = 0; i < cap_tokens; i++) slots[i] = -1;
        for (int i = 0; i < cap_segments * table_width; i++) tables[i] = -1;
        for (int i = 0; i < n; i++) {
            const int len = g.table_len[i], p0 = positions[i];
            if (len > table_width) { *err_request = i; return PLLM_PACK_WIDTH; }
            if (p0 + 1 > len * page_size) { *err_request = i; return PLLM_PACK_NO_PAGE; }
            memcpy(tables + (size_t)i * table_width, g.tables[i], (size_t)len * sizeof(int));
            const int page = g.tables[i][p0 / page_size];
            if (page < 0) { *err_request = i; return PLLM_PACK_FREED_PAGE; }
            slots[i] = page * page_size + p0 % page_size;
        }
        if (!g.plans) continue;
        // ---- the attention work items: one tile a request, cut into splits when the step has
        // too few tiles to fill the GPU (kernels/attention_plan.py: plan_attention) -------------
        int* work = out + g.off_work;
        int* red = out + g.off_red;
        int want = 1;
        if ((long long)n * g.ctas_per_item < target_ctas) {
            want = target_ctas / (n * g.ctas_per_item);
            if (want < 2) want = 2;
        }
        int n_work = 0, n_red = 0, parts = 0;
        for (int i = 0; i < n; i++) {
            const int p0 = positions[i];
            const int kv_end = p0 + 1;
            const int kv_begin = g.window > 0 ? (p0 - (g.window - 1) > 0 ? p0 - (g.window - 1) : 0) : 0;
            const int keys = kv_end - kv_begin;
            int splits = 1;
            if (want > 1) {
                splits = keys / min_split_keys < want ? keys / min_split_keys : want;
                if (splits < 1) splits = 1;
                if (splits > MAX_SPLITS) splits = MAX_SPLITS;
            }
            int chunk = ceil_div(ceil_div(keys, splits), SPLIT_ALIGN) * SPLIT_ALIGN;
            const int n_split = splits > 1 ? ceil_div(keys, chunk) : 1;
            const bool is_split = n_split > 1;
            if (n_work + n_split > g.max_work || (is_split && (n_red + 1 > g.max_red || parts + n_split > g.max_parts))) {
                *err_request = i;
                return PLLM_PACK_WORK;
            }
            for (int k = 0; k < n_split; k++) {
                int* w = work + 8 * (n_work + k);
                const int begin = kv_begin + k * chunk;
                w[0] = i; w[1] = i; w[2] = 1; w[3] = p0;
                w[4] = begin;
                w[5] = is_split ? (begin + chunk < kv_end ? begin + chunk : kv_end) : kv_end;
                w[6] = is_split ? parts + k : -1;
                w[7] = is_split ? (n_split << 16) | k : 0;
            }
            if (is_split) {
                int* r = red + 4 * n_red;
                r[0] = i; r[1] = parts; r[2] = n_split; r[3] = 1;
                n_red++;
                parts += n_split;
            }
            n_work += n_split;
        }
        out[g.off_n_work] = n_work;
        out[g.off_n_red] = n_red;
    }
    return PLLM_OK;
}
