// C names for the host-side rules of host_rules.h, for callers that are not C++ (the Python engine through ctypes).
// No CUDA: this file builds with the host compiler alone.
#include "host_rules.h"

#define JK_HOST_EXPORT extern "C" __attribute__((visibility("default")))

// ---- page pool -----------------------------------------------------------------------------------------------
JK_HOST_EXPORT void *jk_pool_create(int num_pages, int reserved) {
    if (num_pages <= reserved || reserved < 0) return nullptr;
    return new jk::PagePool(num_pages, reserved);
}
JK_HOST_EXPORT void jk_pool_destroy(void *pool) { delete static_cast<jk::PagePool *>(pool); }
JK_HOST_EXPORT int jk_pool_alloc(void *pool, int n, int *out) { return static_cast<jk::PagePool *>(pool)->alloc(n, out) ? 0 : 1; }
JK_HOST_EXPORT int jk_pool_free(void *pool, const int *pages, int n) { return static_cast<jk::PagePool *>(pool)->free(pages, n); }
JK_HOST_EXPORT int jk_pool_available(const void *pool) { return static_cast<const jk::PagePool *>(pool)->available(); }
JK_HOST_EXPORT int jk_pool_high_water(const void *pool) { return static_cast<const jk::PagePool *>(pool)->high_water(); }
JK_HOST_EXPORT int jk_pool_is_held(const void *pool, int page) { return static_cast<const jk::PagePool *>(pool)->is_held(page) ? 1 : 0; }

// ---- a step's metadata ---------------------------------------------------------------------------------------
JK_HOST_EXPORT int jk_max_cache_groups() { return jk::MAX_CACHE_GROUPS; }
JK_HOST_EXPORT int jk_max_step_lists() { return jk::MAX_STEP_LISTS; }
// offsets[0..6]: tokens, positions, row_req, want_rows, req_start, req_pos, slot_ids; then one per cache group; then the
// offset of the extra words; returns the total number of words
JK_HOST_EXPORT int jk_step_layout(int T, int B, int n_groups, int max_blocks, int extra_words, int *offsets) {
    const jk::StepLayout lay(T, B, n_groups, max_blocks, extra_words);
    const int base[7] = {lay.tokens, lay.positions, lay.row_req, lay.want_rows, lay.req_start, lay.req_pos, lay.slot_ids};
    if (offsets) {
        for (int i = 0; i < 7; ++i) offsets[i] = base[i];
        for (int g = 0; g < jk::MAX_CACHE_GROUPS; ++g) offsets[7 + g] = lay.tables[g];
        offsets[7 + jk::MAX_CACHE_GROUPS] = lay.extra;
    }
    return lay.total;
}
// zeroes the buffer's words and packs the batch; returns the number of rows
JK_HOST_EXPORT int jk_pack_step(int *host, int T_padded, int B, int pad_B, int extra_words, const int *tokens, const int *lens,
                                const int *starts, const int *slots, const int *want, int n_want, int n_groups, int max_blocks,
                                const int *const *tables) {
    const jk::StepLayout lay(T_padded, pad_B, n_groups, max_blocks, extra_words);
    memset(host, 0, sizeof(int) * (size_t)lay.total);
    return jk::pack_step(host, lay, B, pad_B, tokens, lens, starts, slots, want, n_want, n_groups, max_blocks, tables);
}

// ---- the attention mixer's work lists ---------------------------------------------------------------------------
JK_HOST_EXPORT int jk_attention_short_rows() { return jk::SHORT_ROWS; }
JK_HOST_EXPORT int jk_attention_tile_rows() { return jk::TILE_ROWS; }
JK_HOST_EXPORT int jk_attention_short_rows_capacity(int T) { return jk::attention_short_rows_capacity(T); }
JK_HOST_EXPORT int jk_attention_tiles_capacity(int T, int B) { return jk::attention_tiles_capacity(T, B); }
// counts[0..1]: short rows, tiles
JK_HOST_EXPORT void jk_attention_work_lists(int B, int pad_B, const int *lens, const int *starts, int *short_rows, int *tiles,
                                            int *counts) {
    const jk::AttentionLists c = jk::attention_work_lists(B, pad_B, lens, starts, short_rows, tiles);
    counts[0] = c.n_short; counts[1] = c.n_tiles;
}

// ---- attention cuts, product routes, tables, uniforms -----------------------------------------------------------
JK_HOST_EXPORT int jk_decode_splits(int nrows, int nkvh, int group, int keys, int sms, int dh) {
    return jk::decode_splits(nrows, nkvh, group, keys, sms, dh);
}
JK_HOST_EXPORT long long jk_decode_scratch_floats(int nrows, int nh, int dh, int splits) {
    return jk::decode_scratch_floats(nrows, nh, dh, splits);
}
JK_HOST_EXPORT int jk_decode_keys_hint(int context, int window) { return jk::decode_keys_hint(context, window); }
JK_HOST_EXPORT int jk_attention_tcgen05_takes(int dh, int page_size) { return jk::attention_tcgen05_takes(dh, page_size) ? 1 : 0; }
JK_HOST_EXPORT int jk_context_bucket(int longest, int max_positions) { return jk::context_bucket(longest, max_positions); }
// routing[0..5]: sms, tcgen05_min_rows, tcgen05_min_tiles, tcgen05_min_fill_pct, skinny_min_blocks, library_only
static jk::Routing routing_of(const int *v) {
    jk::Routing r;
    r.sms = v[0]; r.tcgen05_min_rows = v[1]; r.tcgen05_min_tiles = v[2]; r.tcgen05_min_fill_pct = v[3];
    r.skinny_min_blocks = v[4]; r.library_only = v[5];
    return r;
}
JK_HOST_EXPORT int jk_product_route(const int *routing, int rows, int n, int k, int kind, int small_ok, int tcgen05_ok) {
    return (int)jk::product_route(routing_of(routing), rows, n, k, kind, small_ok != 0, tcgen05_ok != 0);
}
JK_HOST_EXPORT int jk_takes_tcgen05(const int *routing, int rows, int n, int k) {
    return jk::takes_tcgen05(routing_of(routing), rows, n, k) ? 1 : 0;
}
JK_HOST_EXPORT void jk_rotary_tables(double theta, int half, int positions, double angle_scale, float *cos_out, float *sin_out) {
    jk::rotary_tables(theta, half, positions, angle_scale, cos_out, sin_out);
}
JK_HOST_EXPORT float jk_uniform_for(unsigned long long seed, unsigned long long index) { return jk::uniform_for(seed, index); }
