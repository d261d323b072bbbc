// Rules of the engine that run on the host and that more than one part of it follows, each written ONCE.
//
// Plain C++ without CUDA: the Python engine calls them through libjk_host.so (host.cpp gives them C names), the native
// step (runner.cu) and the C interface (capi.cu) include this header.  What lives here:
//   - the page pool behind a cache group (which pages are free, last freed first, never page 0);
//   - the layout of a step's metadata buffer and the packing of a batch into it;
//   - the attention mixer's work lists (rows of requests that bring few rows, tiles of the others);
//   - how many ways the decode attention cuts a row's keys;
//   - which kernel takes a bfloat16 product of a given shape;
//   - the rotary tables;
//   - the uniform number for the token at a position of a request.
#pragma once

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

namespace jk {

// ---- the page pool ---------------------------------------------------------------------------------------------
// Pages are handed out last-freed-first, so a page that a finished request gave back is the next one to be used
// again.  The first `reserved` pages are never handed out; page 0 is the null page that padding rows read and write.
class PagePool {
  public:
    PagePool(int num_pages, int reserved) : num_pages_(num_pages), reserved_(reserved), held_((size_t)num_pages, 0) {
        free_.reserve((size_t)num_pages);
        for (int p = num_pages - 1; p >= reserved; --p) free_.push_back(p);      // the lowest page goes out first
    }
    int capacity() const { return num_pages_ - reserved_; }
    int available() const { return (int)free_.size(); }
    int in_use() const { return capacity() - available(); }
    int high_water() const { return high_water_; }
    int num_pages() const { return num_pages_; }
    int reserved() const { return reserved_; }
    // n pages into out; false (and nothing taken) if fewer are free
    bool alloc(int n, int *out) {
        if (n < 0 || n > (int)free_.size()) return false;
        for (int i = 0; i < n; ++i) {
            out[i] = free_.back();
            free_.pop_back();
            held_[(size_t)out[i]] = 1;
        }
        high_water_ = std::max(high_water_, in_use());
        return true;
    }
    // 0 ok; 1 a page that is not this pool's; 2 a page that is not out (freed twice); 3 a page twice in one call.
    // Nothing is freed unless all of them can be.
    int free(const int *pages, int n) {
        for (int i = 0; i < n; ++i) {
            if (pages[i] < reserved_ || pages[i] >= num_pages_) return 1;
            if (!held_[(size_t)pages[i]]) return 2;
        }
        for (int i = 0; i < n; ++i) {
            if (held_[(size_t)pages[i]] == 2) {
                for (int j = 0; j < i; ++j) held_[(size_t)pages[j]] = 1;
                return 3;
            }
            held_[(size_t)pages[i]] = 2;
        }
        for (int i = 0; i < n; ++i) {
            held_[(size_t)pages[i]] = 0;
            free_.push_back(pages[i]);
        }
        return 0;
    }
    bool is_held(int page) const { return page >= 0 && page < num_pages_ && held_[(size_t)page] != 0; }

  private:
    int num_pages_, reserved_, high_water_ = 0;
    std::vector<int> free_;
    std::vector<unsigned char> held_;
};

// ---- a step's metadata -----------------------------------------------------------------------------------------
constexpr int MAX_CACHE_GROUPS = 8;
constexpr int MAX_STEP_LISTS = 8;

inline int align4(int n) { return (n + 3) & ~3; }

// Offsets (in 32-bit words) of a step's arrays inside the one buffer that is copied to the device per step: what
// every model needs (tokens, positions, the request of each row, the wanted rows, each request's first row, first
// position and state slot, a block table per cache group), then `extra_words` for the work lists that the model's
// mixers ask for (see attention_work_lists below for this architecture's).
struct StepLayout {
    int tokens, positions, row_req, want_rows, req_start, req_pos, slot_ids;
    int tables[MAX_CACHE_GROUPS];
    int extra, total;
    StepLayout(int T, int B, int n_groups, int max_blocks, int extra_words) {
        int o = 0;
        tokens = o; o += align4(T);
        positions = o; o += align4(T);
        row_req = o; o += align4(T);
        want_rows = o; o += align4(T);
        req_start = o; o += align4(B + 1);
        req_pos = o; o += align4(B);
        slot_ids = o; o += align4(B);
        for (int g = 0; g < MAX_CACHE_GROUPS; ++g) {
            tables[g] = o;
            if (g < n_groups) o += align4(B * max_blocks);
        }
        extra = o; o += align4(extra_words);
        total = o;
    }
};

// Packs a batch of B requests (request i brings lens[i] tokens that start at position starts[i]; padded to pad_B
// requests by requests of one row that use slot 0 and the null page at position 0) into `host`, which holds
// `lay.total` zeroed words.  `tables[g]` is [B, max_blocks] page ids, or null (then the caller fills that table);
// `want` lists the wanted places as row indices of the whole step.  Returns the number of rows.
inline int pack_step(int *host, const StepLayout &lay, int B, int pad_B, const int *tokens, const int *lens, const int *starts,
                     const int *slots, const int *want, int n_want, int n_groups, int max_blocks, const int *const *tables) {
    int row = 0;
    for (int i = 0; i < B; ++i) {
        const int n = lens[i], s = starts[i];
        host[lay.req_start + i] = row;
        host[lay.req_pos + i] = s;
        host[lay.slot_ids + i] = slots ? slots[i] : 0;
        for (int t = 0; t < n; ++t) {
            host[lay.tokens + row + t] = tokens[row + t];
            host[lay.positions + row + t] = s + t;
            host[lay.row_req + row + t] = i;
        }
        row += n;
    }
    for (int i = B; i < pad_B; ++i) {       // padding rows of a captured step
        host[lay.req_start + i] = row;
        host[lay.row_req + row] = i;
        ++row;
    }
    host[lay.req_start + pad_B] = row;
    for (int i = 0; i < n_want; ++i) host[lay.want_rows + i] = want[i];
    for (int g = 0; g < n_groups; ++g)
        if (tables && tables[g]) memcpy(host + lay.tables[g], tables[g], sizeof(int) * (size_t)B * max_blocks);
    return row;
}

// ---- the attention mixer's work lists ------------------------------------------------------------------------------
// The softmax attention of this architecture treats requests that bring few rows to a step and requests that bring
// many differently: a request with at most SHORT_ROWS rows goes to the split-key decode kernels row by row; the rows of
// the others are cut into tiles of TILE_ROWS query rows for the prefill kernels.  Its two lists: the short rows, and
// (request, first row) of every tile, the tiles that see the most keys first (the kernels start tiles in list order).
constexpr int SHORT_ROWS = 8;
constexpr int TILE_ROWS = 128;
inline int attention_short_rows_capacity(int T) { return align4(T); }
inline int attention_tiles_capacity(int T, int B) { return align4(2 * (T / TILE_ROWS + B)); }
struct AttentionLists {
    int n_short, n_tiles;
};
inline AttentionLists attention_work_lists(int B, int pad_B, const int *lens, const int *starts, int *short_rows, int *tiles) {
    struct Tile { int keys, req, row; };
    std::vector<Tile> found;
    AttentionLists c{0, 0};
    int row = 0;
    for (int i = 0; i < B; ++i) {
        const int n = lens[i];
        if (n <= SHORT_ROWS)
            for (int t = 0; t < n; ++t) short_rows[c.n_short++] = row + t;
        else
            for (int t0 = 0; t0 < n; t0 += TILE_ROWS) found.push_back({starts[i] + t0, i, row + t0});
        row += n;
    }
    for (int i = B; i < pad_B; ++i) short_rows[c.n_short++] = row++;
    std::stable_sort(found.begin(), found.end(), [](const Tile &a, const Tile &b) { return a.keys > b.keys; });
    for (size_t t = 0; t < found.size(); ++t) {
        tiles[2 * t] = found[t].req;
        tiles[2 * t + 1] = found[t].row;
    }
    c.n_tiles = (int)found.size();
    return c;
}

// ---- how many ways the decode attention cuts each row's key range ------------------------------------------------
// It depends on the batch's size and on `keys`, the context length the step is planned for (a captured step keeps
// its grid, so the caller passes a bucket of the live lengths, not the lengths themselves).
// Head sizes 64 and 128 (the tensor-core kernel: a block per row, key/value head and up to 16 query heads, two blocks
// an SM), from measurements on the 1B, 2B and 8B shapes: as many cuts as make the blocks fill the SMs once (rounded),
// as long as a block keeps 256 keys; then further, up to two rounds of blocks, as long as a block keeps 1024 keys (a
// block's fixed part costs about as much as a few hundred keys, and blocks that all start and end together read
// slower than blocks that overlap).  Other head sizes (the kernel of the CUDA cores, three blocks an SM): the choice
// weighs full waves of blocks against a block's fixed cost of about 128 keys' worth of time.
inline int decode_splits(int nrows, int nkvh, int group, int keys, int sms, int dh) {
    keys = std::max(1, keys);
    if (dh == 64 || dh == 128) {
        const long long blocks = std::max(1, nrows * nkvh * ((group + 15) / 16));
        const long long slots = 2LL * sms;
        long long s = std::max(1LL, std::min({(2 * slots + blocks) / (2 * blocks), (long long)keys / 256, 32LL}));
        while (blocks * (s + 1) <= 2 * slots && keys / (s + 1) >= 1024 && s < 32) ++s;
        // heads of 128: a launch of at most one block an SM runs blocks of eight warps, which pass keys twice as fast;
        // half the cuts is then better than two rounds of the narrow blocks (16 rows x 4,096 keys, 2 key/value heads:
        // 18.3 against 21.5 us)
        if (dh == 128 && blocks * s > sms && blocks * (s / 2) <= sms && s >= 2) s /= 2;
        return (int)s;
    }
    const long long blocks = std::max(1, nrows * nkvh * (group > 4 ? (group + 3) / 4 : 1));
    const long long slots = (long long)sms * 3;
    int best = 1;
    double best_cost = -1;
    for (int s = 1; s <= 32; ++s) {
        if (s > 1 && (double)keys / s < 64) break;
        const long long waves = (blocks * s + slots - 1) / slots;
        const double cost = waves * (128 + (double)keys / s);
        if (best_cost < 0 || cost < best_cost * 0.97) best = s, best_cost = cost;      // fewer cuts unless clearly better
    }
    return best;
}
// `keys` for a row that sees at most `window` keys (0: all) of a context planned for `context` positions: half of what a
// row can see stands for the lengths (the thresholds above were measured with that convention).
inline int decode_keys_hint(int context, int window) {
    const int reach = window > 0 ? std::min(window, context) : context;
    return std::max(1, reach / 2);
}
// floats of scratch that `splits` cuts of `nrows` rows need (partial outputs, maxima and sums); none for one cut
inline long long decode_scratch_floats(int nrows, int nh, int dh, int splits) {
    return splits <= 1 ? 0 : (long long)nrows * nh * splits * (dh + 2);
}
// The context length a step is planned for: the longest live request rounded up to a power of two, at least 4,096, at
// most the model's maximum.  Captured decode steps are kept per (batch bucket, this bucket), so a model with a context of
// 32k that serves short requests cuts their keys as a model of 4k would.  (Below 4,096 the measured optimum does not move:
// at 512 keys, batch 1 and 8, the cuts chosen for 4,096 are 3 % faster than those chosen for 1,024.)
inline int context_bucket(int longest, int max_positions) {
    int b = 4096;
    while (b < longest && b < max_positions) b *= 2;
    return std::min(b, std::max(1, max_positions));
}

// Head and page sizes for which the tcgen05 prefill attention is built (the page must divide a tile of 128 keys and
// fill whole groups of 8 swizzled rows).
inline bool attention_tcgen05_takes(int dh, int page_size) {
    return (dh == 64 || dh == 128) && (page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64 || page_size == 128);
}

// ---- which kernel takes a bfloat16 product ------------------------------------------------------------------------
struct Routing {
    int sms = 148;
    int tcgen05_min_rows = 129, tcgen05_min_tiles = 200, tcgen05_min_fill_pct = 80;     // measured: see takes_tcgen05
    int skinny_min_blocks = 0;        // fewest blocks for the few-rows tcgen05 kernel (0: one per SM)
    int library_only = 0;             // 1: every bfloat16 product goes to the library
};
enum ProductKind { PRODUCT_F32 = 0, PRODUCT_RESIDUAL = 1, PRODUCT_SWIGLU = 2 };
enum Route { ROUTE_LIBRARY = 0, ROUTE_SMALL = 1, ROUTE_SKINNY = 2, ROUTE_TCGEN05 = 3 };

// Whether the tiled tcgen05 product takes `rows` x `n` over `k`.  Measured on the 1B, 2B and 8B shapes, whole steps of
// 160 to 2,048 rows against the library's product with separate elementwise kernels: from `min_rows` rows on, a product
// with at least `min_tiles` output tiles of 128 x 128 whose rows fill their tiles of 128 to `min_fill_pct` per cent is
// as fast or faster on the tcgen05 kernel (fused epilogues, dependent launch, cuts of K for the products that add into
// the residual stream); products of fewer tiles go to the library, whose smaller tiles fill the SMs better.  Very wide
// outputs (the logits) are taken from 17 rows.
inline bool takes_tcgen05(const Routing &r, int rows, int n, int k) {
    if (r.library_only || rows <= 16 || k < 8 || k % 8) return false;
    const long long row_tiles = (rows + 127) / 128;
    if (row_tiles * ((n + 255) / 256) >= 3LL * r.sms) return true;
    if (rows < r.tcgen05_min_rows || rows * 100LL < (long long)r.tcgen05_min_fill_pct * row_tiles * 128) return false;
    return row_tiles * ((n + 127) / 128) >= r.tcgen05_min_tiles;
}
// Blocks that the few-rows tcgen05 kernel starts for a product with `n` output features over `k`: tiles of 128 features
// (64 for SwiGLU, whose tile holds as many up rows again); a product that is added into the residual stream splits K
// until the blocks fill the SMs twice, as long as a block keeps 8 steps of 64.
inline long long skinny_blocks(int sms, int n, int k, int kind) {
    const int nk = (k + 63) / 64;
    if (kind == PRODUCT_SWIGLU) return (n + 63) / 64;
    const int tiles = (n + 127) / 128;
    int splits = 1;
    if (kind == PRODUCT_RESIDUAL) splits = std::max(1, std::min(2 * sms / tiles, nk / 8));
    const int ksteps = (nk + splits - 1) / splits;
    return (long long)tiles * ((nk + ksteps - 1) / ksteps);
}
// Which kernel takes a product of `rows` rows: up to 128 rows the few-rows tcgen05 kernel once it has a block for every
// SM (it then reads W at 5 to 6 TB/s), always once it has four blocks for every SM; up to 16 rows the small-row kernel
// (if it takes the shape: `small_ok`) where it
// has a second block on the SM to overlap its load phase with (a slice of 16 rows x K fits twice), or so few tiles that
// they make one wave, or nothing better; above that the tiled tcgen05 kernel by the rule above; else the library.
// `tcgen05_ok`: the tcgen05 module is there.
inline Route product_route(const Routing &r, int rows, int n, int k, int kind, bool small_ok, bool tcgen05_ok) {
    if (r.library_only) return ROUTE_LIBRARY;
    if (rows <= 128) {
        const long long need = r.skinny_min_blocks > 0 ? r.skinny_min_blocks : r.sms;
        const bool skinny = tcgen05_ok && k >= 8 && k % 8 == 0 && skinny_blocks(r.sms, n, k, kind) >= need;
        // a very wide output (the logits): with four rounds of blocks and more the few-rows tcgen05 kernel reads W at 0.95 of
        // the copy bandwidth for any row count (2B, 1B and 8B output matrices at 1, 8 and 16 rows: 91, 38 and 92 us against
        // 132, 50 and 211 us of the small-row kernel at 8 rows)
        if (skinny && skinny_blocks(r.sms, n, k, kind) >= 4LL * r.sms) return ROUTE_SKINNY;
        if (rows <= 16 && small_ok) {
            const long long out_rows = kind == PRODUCT_SWIGLU ? 2LL * n : n;
            if (!skinny || 2 * (32LL * k + 8192) <= 227 * 1024 || (out_rows + 15) / 16 <= r.sms) return ROUTE_SMALL;
        }
        if (skinny) return ROUTE_SKINNY;
    }
    if (tcgen05_ok && takes_tcgen05(r, rows, n, k)) return ROUTE_TCGEN05;
    return ROUTE_LIBRARY;
}

// ---- rotary tables --------------------------------------------------------------------------------------------
// Angle of pair j at position p: p / theta^(j / half), computed in double and rounded once to float32.
inline void rotary_tables(double theta, int half, int positions, double angle_scale, float *cos_out, float *sin_out) {
    std::vector<double> inv((size_t)half);
    for (int j = 0; j < half; ++j) inv[(size_t)j] = angle_scale * std::pow(theta, -((double)j / half));
    for (int p = 0; p < positions; ++p)
        for (int j = 0; j < half; ++j) {
            const double a = (double)p * inv[(size_t)j];
            cos_out[(size_t)p * half + j] = (float)std::cos(a);
            sin_out[(size_t)p * half + j] = (float)std::sin(a);
        }
}

// ---- the uniform number of a drawn token ---------------------------------------------------------------------------
// A float in [0, 1) from (seed, absolute position of the new token): the splitmix64 finaliser, top 24 bits.  It does
// not depend on what else is in the batch or on how the prompt was cut.
inline float uniform_for(uint64_t seed, uint64_t index) {
    uint64_t z = seed * 0x9E3779B97F4A7C15ull + (index + 1) * 0xBF58476D1CE4E5B9ull;
    z ^= z >> 30;
    z *= 0xBF58476D1CE4E5B9ull;
    z ^= z >> 27;
    z *= 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (float)(z >> 40) / (float)(1 << 24);
}

}  // namespace jk
