// C ABI of libftq_b200.so: argument checking, table packing and kernel dispatch.
// Every entry point is declared (with the reference interface it replaces) in
// include/ftq_b200.h.
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cfloat>
#include <atomic>
#include <cstdint>
#include <cstring>
#include <random>
#include <cstdlib>
#include <mutex>

#include "../../include/ftq_b200.h"
#include "ftq_dense.cuh"
#include "ftq_launch.h"
#include "ftq_tq_v1_launch.h"

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int cuda_fail(cudaError_t e, const char* what) {
    return fail(FTQ_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

bool dim_ok(int d) { return d == 64 || d == 128 || d == 256; }
bool bits_ok(int b) { return b >= 2 && b <= 4; }
bool dtype_ok(int t) { return t == FTQ_F32 || t == FTQ_F16 || t == FTQ_BF16; }
size_t dtype_size(int t) { return t == FTQ_F32 ? 4 : 2; }
bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// signs must be exactly +-1: the kernels flip the sign bit instead of multiplying.
int pack_signs(const float* signs_host, int d, ftq::SignBits* out) {
    memset(out, 0, sizeof(*out));
    if (!signs_host) return FTQ_OK;
    for (int i = 0; i < d; i++) {
        const float s = signs_host[i];
        if (s == -1.0f) out->w[i >> 5] |= 1u << (i & 31);
        else if (s != 1.0f) return fail(FTQ_ERR_INVALID, "signs[%d] = %g is not +1 or -1", i, s);
    }
    return FTQ_OK;
}

int pack_levels(const float* levels_host, int bits, ftq::Codebook* out) {
    if (!levels_host) return fail(FTQ_ERR_INVALID, "levels table is NULL");
    memset(out, 0, sizeof(*out));
    for (int i = 0; i < (1 << bits); i++) out->v[i] = levels_host[i];
    return FTQ_OK;
}

float rsqrt_dim(int d) { return static_cast<float>(std::pow(static_cast<double>(d), -0.5)); }

int make_encode_tables(int d, int bits, const float* signs_host, const float* boundaries_host,
                       ftq::EncodeTables* tab) {
    if (!boundaries_host) return fail(FTQ_ERR_INVALID, "boundaries table is NULL");
    const int nb = (1 << bits) + 1;
    for (int i = 1; i < nb; i++)
        if (!(boundaries_host[i - 1] <= boundaries_host[i]))
            return fail(FTQ_ERR_INVALID, "boundaries must be ascending");
    memset(tab, 0, sizeof(*tab));
    const int rc = pack_signs(signs_host, d, &tab->signs);
    if (rc) return rc;
    // code = clamp(#{b < x} - 1, 0, 2^bits - 1) = #{interior boundaries < x}
    for (int j = 1; j < nb - 1; j++) tab->bounds[j - 1] = boundaries_host[j];
    tab->rsqrt_d = rsqrt_dim(d);
    return FTQ_OK;
}

// Table quantizer of the throughput encode kernel: x is mapped to a cell of [-1, 1] by
// the same single-precision FMA the kernel uses; usable when no cell holds two boundaries
// and no boundary is so close to zero that a 2^100 scaling cannot separate it from x.
uint32_t quant_cell(float x) {
    const float v = fmaf(x, ftq::kCellScale, ftq::kCellMagic);
    uint32_t bits;
    memcpy(&bits, &v, 4);
    return (bits & 0xFF80u) >> 7;
}

bool make_encode2_tables(const ftq::EncodeTables& tab, int bits, ftq::Encode2Tables* out) {
    const int nb = (1 << bits) - 1;  // interior boundaries, ascending
    out->signs = tab.signs;
    out->rsqrt_d = tab.rsqrt_d;
    for (int c = 0; c < ftq::kQuantCells; c++) {
        out->cells[c].neg_thr_scaled = -FLT_MAX;
        out->cells[c].base = 0.f;
    }
    uint32_t prev = 0xffffffffu;
    for (int j = 0; j < nb; j++) {
        const float b = tab.bounds[j];
        if (!(b > -1.0f && b < 1.0f) || (j > 0 && !(tab.bounds[j - 1] < b))) return false;
        if (std::fabs(b) < 1e-20f) return false;
        const uint32_t c = quant_cell(b);
        if (c == prev || c >= static_cast<uint32_t>(ftq::kQuantCells)) return false;
        prev = c;
        out->cells[c].neg_thr_scaled = -b * ftq::kStepScale;
        for (uint32_t k = c + 1; k < static_cast<uint32_t>(ftq::kQuantCells); k++)
            out->cells[k].base += 1.f;
    }
    return true;
}

cudaError_t dispatch_encode(int d, int bits, int dtype, const ftq::EncodeSource& src_in,
                            const ftq::EncodeSink& sink_in, const ftq::EncodeTables& tab,
                            int64_t n_vec, int n_layers, cudaStream_t st) {
    // vector indices are split into (token, head) with 31-bit arithmetic in the kernels (the
    // public entry points reject larger counts, which no resident input can reach)
    if (n_vec >= (1ll << 31) || src_in.n_inner <= 0 || sink_in.Hkv <= 0) return cudaErrorInvalidValue;
    ftq::EncodeSource src = src_in;
    ftq::EncodeSink sink = sink_in;
    src.div_inner = ftq::make_fastdiv(static_cast<uint32_t>(src.n_inner));
    sink.div_hkv = ftq::make_fastdiv(static_cast<uint32_t>(sink.Hkv));
    // A handful of vectors (a decode step) is launch-bound either way: the simple kernel
    // skips the table set-up.  Bulk encodes take the throughput kernel when the codebook allows.
    ftq::Encode2Tables tab2;
    const bool fast = n_vec >= 2048 && make_encode2_tables(tab, bits, &tab2);
    const ftq::Encode2Tables* t2 = fast ? &tab2 : nullptr;
    switch (d) {
        case 64: return ftq::launch_encode_d64(bits, dtype, src, sink, tab, t2, n_vec, n_layers, st);
        case 128: return ftq::launch_encode_d128(bits, dtype, src, sink, tab, t2, n_vec, n_layers, st);
        case 256: return ftq::launch_encode_d256(bits, dtype, src, sink, tab, t2, n_vec, n_layers, st);
    }
    return cudaErrorInvalidValue;
}

// fp32 -> fp16 -> fp32 with round to nearest even (host side).
float round_to_half(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = x & 0x80000000u;
    uint32_t a = x & 0x7fffffffu;
    if (a >= 0x477ff000u) a = 0x7f800000u;           // overflow -> inf
    else if (a < 0x38800000u) {                      // half subnormal range: quantum 2^-24
        float v;
        memcpy(&v, &a, 4);
        v = std::nearbyint(v * 16777216.0f) / 16777216.0f;
        memcpy(&a, &v, 4);
    } else {
        const uint32_t rem = a & 0x1fffu;
        a &= ~0x1fffu;
        if (rem > 0x1000u || (rem == 0x1000u && (a & 0x2000u))) a += 0x2000u;
    }
    a |= sign;
    float r;
    memcpy(&r, &a, 4);
    return r;
}

// Factor s in [1, 2) for the V centroids of the tensor-core path: fp16(s * level) / s should
// have no common bias.  The bias is weighted with the cell probabilities of N(0, 1/D) (cell
// edges = level midpoints); a small share of the mean absolute error keeps s from trading a
// zero bias against large individual errors.
float search_v_scale(const float* levels, int bits, int head_dim);

// The search costs ~1 ms of host time: results are remembered per (levels, bits, head_dim).
float choose_v_scale(const float* levels, int bits, int head_dim) {
    struct Entry { float levels[16]; int bits, head_dim; float scale; };
    static std::mutex mu;
    static Entry cache[16];
    static int n_cached = 0, next_slot = 0;
    const size_t nbytes = sizeof(float) << bits;
    {
        std::lock_guard<std::mutex> lock(mu);
        for (int i = 0; i < n_cached; i++)
            if (cache[i].bits == bits && cache[i].head_dim == head_dim &&
                memcmp(cache[i].levels, levels, nbytes) == 0)
                return cache[i].scale;
    }
    const float sc = search_v_scale(levels, bits, head_dim);
    std::lock_guard<std::mutex> lock(mu);
    Entry& e = cache[next_slot];
    memset(&e, 0, sizeof(e));
    memcpy(e.levels, levels, nbytes);
    e.bits = bits; e.head_dim = head_dim; e.scale = sc;
    next_slot = (next_slot + 1) % 16;
    if (n_cached < 16) n_cached++;
    return sc;
}

float search_v_scale(const float* levels, int bits, int head_dim) {
    const int n = 1 << bits;
    double prob[16];
    const double inv_sigma = std::sqrt(static_cast<double>(head_dim));
    double prev = 0.0;
    for (int c = 0; c < n; c++) {
        const double cdf = c == n - 1 ? 1.0
            : 0.5 * std::erfc(-0.5 * (static_cast<double>(levels[c]) + levels[c + 1]) * inv_sigma /
                              std::sqrt(2.0));
        prob[c] = cdf - prev;
        prev = cdf;
    }
    float best = 1.0f;
    double best_cost = 1e30;
    for (int i = 0; i < 8192; i++) {
        const float sc = 1.0f + static_cast<float>(i) / 8192.0f;
        double bias = 0.0, mad = 0.0;
        for (int c = 0; c < n; c++) {
            const double err = static_cast<double>(round_to_half(levels[c] * sc)) / sc - levels[c];
            bias += prob[c] * err;
            mad += prob[c] * std::fabs(err);
        }
        const double cost = std::fabs(bias) + 0.05 * mad;
        if (cost < best_cost) { best_cost = cost; best = sc; }
    }
    return best;
}

// Factor s in [1, 2) for the K centroids of the tensor-core path: the key scores are sums of
// q * centroid products, so what matters there is the SIZE of the centroids' fp16 rounding errors,
// not their common bias: s minimises the probability-weighted mean square of
// fp16(s * level) / s - level (cell probabilities of N(0, 1/D), cell edges = level midpoints).
// 1 / s goes into the softmax scale, so the kernel needs nothing for it.
float choose_k_scale(const float* levels, int bits, int head_dim) {
    struct Entry { float levels[16]; int bits, head_dim; float scale; };
    static std::mutex mu;
    static Entry cache[16];
    static int n_cached = 0, next_slot = 0;
    const size_t nbytes = sizeof(float) << bits;
    {
        std::lock_guard<std::mutex> lock(mu);
        for (int i = 0; i < n_cached; i++)
            if (cache[i].bits == bits && cache[i].head_dim == head_dim &&
                memcmp(cache[i].levels, levels, nbytes) == 0)
                return cache[i].scale;
    }
    const int n = 1 << bits;
    double prob[16];
    const double inv_sigma = std::sqrt(static_cast<double>(head_dim));
    double prev = 0.0;
    for (int c = 0; c < n; c++) {
        const double cdf = c == n - 1 ? 1.0
            : 0.5 * std::erfc(-0.5 * (static_cast<double>(levels[c]) + levels[c + 1]) * inv_sigma /
                              std::sqrt(2.0));
        prob[c] = cdf - prev;
        prev = cdf;
    }
    float best = 1.0f;
    double best_cost = 1e30;
    for (int i = 0; i < 8192; i++) {
        const float sc = 1.0f + static_cast<float>(i) / 8192.0f;
        double mse = 0.0;
        for (int c = 0; c < n; c++) {
            const double err = static_cast<double>(round_to_half(levels[c] * sc)) / sc - levels[c];
            mse += prob[c] * err * err;
        }
        if (mse < best_cost) { best_cost = mse; best = sc; }
    }
    std::lock_guard<std::mutex> lock(mu);
    Entry& e = cache[next_slot];
    memset(&e, 0, sizeof(e));
    memcpy(e.levels, levels, nbytes);
    e.bits = bits; e.head_dim = head_dim; e.scale = best;
    next_slot = (next_slot + 1) % 16;
    if (n_cached < 16) n_cached++;
    return best;
}

struct ChunkPlan {
    int chunk_tokens, n_chunks, n_hpass;
    // tensor-core kernels: units from bulk_units on are cut into tail_chunks chunks of
    // tail_chunk_tokens instead, and the last tail_b_units of them into one chunk more
    // (bulk_units < 0: one split for all units)
    int64_t bulk_units = -1;
    int tail_chunks = 0, tail_chunk_tokens = 0;
    int64_t tail_b_units = 0;
    int tail_b_chunks = 0, tail_b_chunk_tokens = 0;
    int row_chunks() const {
        int m = n_chunks;
        if (tail_chunks > m) m = tail_chunks;
        if (tail_b_units > 0 && tail_b_chunks > m) m = tail_b_chunks;
        return m;
    }
};

// The device-side description of a plan over `units` units (n_regions = 0 for the fp32 kernels'
// single split).
ftq::SplitPlan make_split(const ChunkPlan& pl, int64_t units, bool tensor_core) {
    ftq::SplitPlan sp{};
    if (!tensor_core) return sp;
    auto put = [&](int k, int64_t first_unit, int64_t first_item, int chunks, int tokens) {
        sp.r[k].first_unit = static_cast<int>(first_unit);
        sp.r[k].first_item = static_cast<int>(first_item);
        sp.r[k].chunks = chunks;
        sp.r[k].chunk_tokens = tokens;
        sp.r[k].div_chunks = ftq::make_fastdiv(static_cast<uint32_t>(chunks));
    };
    const int64_t bulk = pl.bulk_units >= 0 ? pl.bulk_units : units;
    put(0, 0, 0, pl.n_chunks, pl.chunk_tokens);
    sp.n_regions = 1;
    int64_t items = bulk * pl.n_chunks;
    if (bulk < units) {
        const int64_t a_units = units - bulk - pl.tail_b_units;
        if (a_units > 0) {
            put(sp.n_regions++, bulk, items, pl.tail_chunks, pl.tail_chunk_tokens);
            items += a_units * pl.tail_chunks;
        }
        if (pl.tail_b_units > 0) {
            put(sp.n_regions++, bulk + a_units, items, pl.tail_b_chunks, pl.tail_b_chunk_tokens);
            items += pl.tail_b_units * pl.tail_b_chunks;
        }
    }
    sp.row_chunks = pl.row_chunks();
    sp.total_items = static_cast<int>(items);
    return sp;
}

// Split the context so that the grid fills the GPU a few times over.
ChunkPlan plan_chunks(int B, int Hq, int Hkv, int d, int max_seq_len, int n_layers) {
    const int gh = 64 / (d / 8);
    const int group = Hq / Hkv;
    ChunkPlan pl;
    pl.n_hpass = (group + gh - 1) / gh;
    const int tile = ftq::kTilePages * ftq::kPageTokens;
    const int64_t units = static_cast<int64_t>(B) * Hkv * pl.n_hpass * n_layers;
    const int64_t target = static_cast<int64_t>(ftq::sm_count()) * 2 * 4;
    const int max_tiles = max_seq_len > 0 ? (max_seq_len + tile - 1) / tile : 1;
    int64_t want = (target + units - 1) / (units > 0 ? units : 1);
    if (want < 1) want = 1;
    if (want > max_tiles) want = max_tiles;
    const int tiles_per_chunk = static_cast<int>((max_tiles + want - 1) / want);
    pl.chunk_tokens = tiles_per_chunk * tile;
    pl.n_chunks = (max_tiles + tiles_per_chunk - 1) / tiles_per_chunk;
    return pl;
}

// Chunking of the tensor-core path (persistent CTAs): few, large chunks keep the per-item
// fixed costs small, more chunks fill the last wave of CTA slots better; the plan with the
// lowest modelled cost wins.  Chunks hold at most 8192 tokens (short enough for the dynamic
// hand-out of items to even out ragged batches; their block ids are staged in shared memory)
// and at least 1024.
// The planner both tensor-core kernels share.  Cost of a plan = waves of items over the CTA slots
// x (pages of an item + the fixed cost of an item, in pages); the cheapest plan wins, the fewest
// chunks among equals.  A plan has up to two regions: as many units as fill whole waves of the
// grid are cut into few, long chunks; the remaining units into more, shorter ones that share the
// last wave.  Items are handed out bulk first, so the short ones also even out the CTAs'
// different speeds.
ChunkPlan plan_two_regions(int64_t units, int64_t slots, int max_seq_len, double item_cost) {
    ChunkPlan pl;
    pl.n_hpass = 1;
    const int seq = max_seq_len > 0 ? max_seq_len : 1;
    const int c_min = (seq + 8191) / 8192;
    const int c_max = (seq + 1023) / 1024 > c_min ? (seq + 1023) / 1024 : c_min;
    auto split = [&](int nc, int* ct, int* real) {
        int t = ((seq + nc - 1) / nc + 63) / 64 * 64;
        if (t > 8192) t = 8192;
        *ct = t;
        *real = (seq + t - 1) / t;
    };
    double best = -1.0;
    for (int nc1 = c_min; nc1 <= c_max && nc1 < c_min + 64; nc1++) {
        int ct1, r1;
        split(nc1, &ct1, &r1);
        const double cost1 = ct1 / 16.0 + item_cost;
        // one split for all units
        const double uniform = static_cast<double>((units * r1 + slots - 1) / slots) * cost1;
        if (best < 0.0 || uniform < best * (1.0 - 1e-9)) {
            best = uniform;
            pl.chunk_tokens = ct1; pl.n_chunks = r1;
            pl.bulk_units = -1; pl.tail_chunks = 0; pl.tail_chunk_tokens = 0;
        }
        // whole waves of this split, the rest of the units cut finer
        const int64_t full = units * r1 / slots;
        const int64_t bulk = full * slots / r1;
        if (full == 0 || bulk >= units) continue;
        for (int nc2 = nc1 + 1; nc2 <= c_max && nc2 <= nc1 + 16; nc2++) {
            int ct2, r2;
            split(nc2, &ct2, &r2);
            if (r2 <= r1) continue;
            const int64_t tail_waves = ((units - bulk) * r2 + slots - 1) / slots;
            const double cost = static_cast<double>(full) * cost1 +
                                static_cast<double>(tail_waves) * (ct2 / 16.0 + item_cost);
            if (cost < best * (1.0 - 1e-9)) {
                best = cost;
                pl.chunk_tokens = ct1; pl.n_chunks = r1;
                pl.bulk_units = bulk; pl.tail_chunks = r2; pl.tail_chunk_tokens = ct2;
            }
        }
    }
    // The CTAs differ in speed by a few percent on identical items (measured), and a last wave
    // with fewer items than CTAs leaves the fastest ones idle.  So some of the tail units get
    // one chunk more, enough for the last wave to hold an item for every CTA: the ticket order
    // hands the longer items to the CTAs that arrive first and the shorter ones to the late ones.
    pl.tail_b_units = 0;
    if (pl.bulk_units >= 0) {
        const int64_t tail_units = units - pl.bulk_units;
        const int64_t items = tail_units * pl.tail_chunks;
        const int64_t missing = (items + slots - 1) / slots * slots - items;
        int ct3, r3;
        split(pl.tail_chunks + 1, &ct3, &r3);
        if (missing > 0 && missing <= tail_units && r3 == pl.tail_chunks + 1 && r3 <= c_max) {
            pl.tail_b_units = missing;
            pl.tail_b_chunks = r3;
            pl.tail_b_chunk_tokens = ct3;
        }
    }
    return pl;
}

// attn_mma_kernel: the fixed cost of an item (publish / fold / next item's queries between
// CTA-wide barriers) weighs about 15 pages for a 16-warp CTA and 30 for an 8-warp one (fitted to
// measured step times of the uniform benchmark shapes).
ChunkPlan plan_chunks_mma(int B, int Hkv, int max_seq_len, int n_layers, int ctas_per_sm) {
    return plan_two_regions(static_cast<int64_t>(B) * Hkv * n_layers,
                            static_cast<int64_t>(ftq::sm_count()) * ctas_per_sm, max_seq_len,
                            ctas_per_sm == 1 ? 15.0 : 30.0);
}

// The streaming kernel.  Measured on B200 (Llama-shaped K4V4 batches of 37..111
// sequences, forced chunk counts): an item costs about 74 pages on top of its own pages (the
// service warps' smaller page share, the publish / fold / prepare hand-overs), so long chunks
// pay -- but whole waves of them rarely match the unit count, hence the two regions.
ChunkPlan plan_chunks_stream(int B, int Hkv, int max_seq_len, int n_layers, int ctas_per_sm) {
    return plan_two_regions(static_cast<int64_t>(B) * Hkv * n_layers,
                            static_cast<int64_t>(ftq::sm_count()) * ctas_per_sm, max_seq_len, 74.0);
}

int attn_mma_stream_ctas(int d, int bits_k, int bits_v, int group) {
    switch (d) {
        case 64: return ftq::attn_mma_stream_ctas_d64(bits_k, bits_v, group);
        case 128: return ftq::attn_mma_stream_ctas_d128(bits_k, bits_v, group);
        case 256: return ftq::attn_mma_stream_ctas_d256(bits_k, bits_v, group);
    }
    return 0;
}

bool use_mma_path(int Hq, int Hkv, int q_dtype) { return Hq / Hkv <= 8 && q_dtype != FTQ_F32; }

size_t partial_bytes(const ChunkPlan& pl, int B, int Hq, int d, int n_layers) {
    return static_cast<size_t>(n_layers) * B * Hq * pl.row_chunks() * (d + 4) * sizeof(float);
}

cudaError_t dispatch_split(int d, int bk, int bv, bool paged, const ftq::AttnParams& p, int n_lb,
                           cudaStream_t st) {
    switch (d) {
        case 64: return ftq::launch_attn_split_d64(bk, bv, paged, p, n_lb, st);
        case 128: return ftq::launch_attn_split_d128(bk, bv, paged, p, n_lb, st);
        case 256: return ftq::launch_attn_split_d256(bk, bv, paged, p, n_lb, st);
    }
    return cudaErrorInvalidValue;
}

cudaError_t dispatch_mma(int d, int bk, int bv, bool shared_lut, const ftq::AttnParams& p, int n_lb,
                         cudaStream_t st, bool* merged) {
    switch (d) {
        case 64: return ftq::launch_attn_mma_d64(bk, bv, shared_lut, p, n_lb, st, merged);
        case 128: return ftq::launch_attn_mma_d128(bk, bv, shared_lut, p, n_lb, st, merged);
        case 256: return ftq::launch_attn_mma_d256(bk, bv, shared_lut, p, n_lb, st, merged);
    }
    return cudaErrorInvalidValue;
}

cudaError_t dispatch_merge(int d, int out_dtype, const float* partials, void* out,
                           const int32_t* seq_lens, int S, int B, int Hq, int Hkv,
                           const ChunkPlan& pl, const ftq::SplitPlan& split, int64_t n_vec,
                           const ftq::SignBits& signs, cudaStream_t st) {
    const float r = rsqrt_dim(d);
    switch (d) {
        case 64:
            return ftq::launch_attn_merge_d64(out_dtype, partials, out, seq_lens, S, B, Hq,
                                              pl.n_chunks, pl.chunk_tokens, n_vec, signs, r, Hkv,
                                              split, st);
        case 128:
            return ftq::launch_attn_merge_d128(out_dtype, partials, out, seq_lens, S, B, Hq,
                                               pl.n_chunks, pl.chunk_tokens, n_vec, signs, r, Hkv,
                                               split, st);
        case 256:
            return ftq::launch_attn_merge_d256(out_dtype, partials, out, seq_lens, S, B, Hq,
                                               pl.n_chunks, pl.chunk_tokens, n_vec, signs, r, Hkv,
                                               split, st);
    }
    return cudaErrorInvalidValue;
}

unsigned grid_for(int64_t n_vec, int vec_per_cta) {
    const int64_t want = (n_vec + vec_per_cta - 1) / vec_per_cta;
    const int64_t cap = static_cast<int64_t>(ftq::sm_count()) * 8;
    return static_cast<unsigned>(want < 1 ? 1 : (want < cap ? want : cap));
}

// ---- v0 gather: one thread per output 32-bit word (codes) or norm
__global__ void v0_gather_kernel(const uint8_t* __restrict__ kv_cache, int64_t num_blocks,
                                 int block_size, int Hkv, int elem_size, int kv_type, int pd,
                                 const int32_t* __restrict__ block_tables, int max_blocks,
                                 const int32_t* __restrict__ seq_lens, int B, int max_seq_len,
                                 uint8_t* __restrict__ out_codes, float* __restrict__ out_norms) {
    const int wpt = pd / 4 + 1;  // words per token-head: codes then the norm
    const int64_t total = static_cast<int64_t>(B) * Hkv * max_seq_len * wpt;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int w = static_cast<int>(i % wpt);
        const int64_t th = i / wpt;  // (b, h, pos)
        const int pos = static_cast<int>(th % max_seq_len);
        const int h = static_cast<int>((th / max_seq_len) % Hkv);
        const int b = static_cast<int>(th / (static_cast<int64_t>(max_seq_len) * Hkv));
        uint32_t val = 0;
        if (pos < seq_lens[b]) {
            const int64_t blk = block_tables[static_cast<int64_t>(b) * max_blocks + pos / block_size];
            const int off = pos % block_size;
            if (static_cast<uint64_t>(blk) < static_cast<uint64_t>(num_blocks)) {
                const uint8_t* slot = kv_cache +
                    ((((static_cast<int64_t>(kv_type) * num_blocks + blk) * block_size + off) * Hkv + h) *
                     elem_size);
                val = *reinterpret_cast<const uint32_t*>(slot + 4 * w);
            } else {
                // a block id outside the cache is never dereferenced: the position's norm reads NaN
                val = w < pd / 4 ? 0u : 0x7fc00000u;
            }
        }
        if (w < pd / 4) reinterpret_cast<uint32_t*>(out_codes + th * pd)[w] = val;
        else out_norms[th] = __uint_as_float(val);
    }
}

}  // namespace

namespace ftq {
int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}
}  // namespace ftq

extern "C" {

int ftq_version(void) { return 100; }

const char* ftq_last_error(void) { return g_err; }

int ftq_packed_dim(int head_dim, int bits) {
    if (head_dim <= 0 || head_dim % 8 || !bits_ok(bits)) return -1;
    return head_dim * bits / 8;
}

int64_t ftq_page_bytes(int head_dim, int bits_k, int bits_v) {
    if (!dim_ok(head_dim) || !bits_ok(bits_k) || !bits_ok(bits_v)) return -1;
    return static_cast<int64_t>(FTQ_PAGE_TOKENS) *
           (ftq::packed_dim(head_dim, bits_k) + ftq::packed_dim(head_dim, bits_v) + 4);
}

int ftq_encode(const void* x, int dtype, int64_t n_vec, int head_dim, int64_t row_stride, int bits,
               const float* signs_host, const float* boundaries_host, uint8_t* packed,
               uint16_t* norms_f16, void* stream) {
    if (!dim_ok(head_dim)) return fail(FTQ_ERR_UNSUPPORTED, "head_dim %d (need 64/128/256)", head_dim);
    if (!bits_ok(bits)) return fail(FTQ_ERR_INVALID, "bits must be 2, 3, or 4, got %d", bits);
    if (!dtype_ok(dtype)) return fail(FTQ_ERR_INVALID, "bad dtype %d", dtype);
    if (n_vec < 0) return fail(FTQ_ERR_INVALID, "n_vec < 0");
    if (n_vec >= (1ll << 31)) return fail(FTQ_ERR_INVALID, "n_vec must be below 2^31 per call");
    if (n_vec == 0) return FTQ_OK;
    if (!x || !packed || !norms_f16) return fail(FTQ_ERR_INVALID, "NULL tensor pointer");
    if (row_stride < head_dim) return fail(FTQ_ERR_INVALID, "row_stride < head_dim");
    if (!aligned(x, 16) || (row_stride * dtype_size(dtype)) % 16)
        return fail(FTQ_ERR_INVALID, "input rows must be 16-byte aligned");
    if (!aligned(packed, 4) || !aligned(norms_f16, 2))
        return fail(FTQ_ERR_INVALID, "outputs must be 4-byte (codes) / 2-byte (norms) aligned");
    ftq::EncodeTables tab;
    int rc = make_encode_tables(head_dim, bits, signs_host, boundaries_host, &tab);
    if (rc) return rc;
    ftq::EncodeSource src{x, 1, row_stride, 0, 0};
    ftq::EncodeSink sink{};
    sink.mode = ftq::kSinkFlat;
    sink.codes = packed;
    sink.norms = norms_f16;
    sink.Hkv = 1;
    cudaError_t e = dispatch_encode(head_dim, bits, dtype, src, sink, tab, n_vec, 1,
                                    static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? FTQ_OK : cuda_fail(e, "ftq_encode launch");
}

int ftq_decode_dense(const uint8_t* packed, const void* norms, int norms_dtype, int64_t n_vec,
                     int head_dim, int bits, const float* levels_host, const float* signs_host,
                     float* out, void* stream) {
    if (!dim_ok(head_dim)) return fail(FTQ_ERR_UNSUPPORTED, "head_dim %d (need 64/128/256)", head_dim);
    if (!bits_ok(bits)) return fail(FTQ_ERR_INVALID, "bits must be 2, 3, or 4, got %d", bits);
    if (norms_dtype != FTQ_F16 && norms_dtype != FTQ_F32)
        return fail(FTQ_ERR_INVALID, "norms must be fp16 or fp32");
    if (n_vec == 0) return FTQ_OK;
    if (!packed || !norms || !out || n_vec < 0) return fail(FTQ_ERR_INVALID, "bad tensor argument");
    if (!aligned(packed, 4) || !aligned(out, 4)) return fail(FTQ_ERR_INVALID, "misaligned tensor");
    ftq::Codebook lv;
    ftq::SignBits sg;
    int rc = pack_levels(levels_host, bits, &lv);
    if (rc) return rc;
    rc = pack_signs(signs_host, head_dim, &sg);
    if (rc) return rc;
    const float r = rsqrt_dim(head_dim);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned grid = grid_for(n_vec, 32);
#define FTQ_DD(DD, BB)                                                                          \
    if (norms_dtype == FTQ_F16)                                                                 \
        ftq::decode_dense_kernel<DD, BB, __half><<<grid, 256, 0, st>>>(                          \
            packed, static_cast<const __half*>(norms), out, lv, sg, r, n_vec);                  \
    else                                                                                        \
        ftq::decode_dense_kernel<DD, BB, float><<<grid, 256, 0, st>>>(                           \
            packed, static_cast<const float*>(norms), out, lv, sg, r, n_vec);
#define FTQ_DB(DD)                                                                              \
    switch (bits) {                                                                             \
        case 2: FTQ_DD(DD, 2) break;                                                            \
        case 3: FTQ_DD(DD, 3) break;                                                            \
        case 4: FTQ_DD(DD, 4) break;                                                            \
    }
    switch (head_dim) {
        case 64: FTQ_DB(64) break;
        case 128: FTQ_DB(128) break;
        case 256: FTQ_DB(256) break;
    }
#undef FTQ_DB
#undef FTQ_DD
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FTQ_OK : cuda_fail(e, "ftq_decode_dense launch");
}

int ftq_rht(const void* x, void* y, int dtype, int64_t n_vec, int head_dim,
            const float* signs_host, int inverse, void* stream) {
    if (!dim_ok(head_dim)) return fail(FTQ_ERR_UNSUPPORTED, "head_dim %d (need 64/128/256)", head_dim);
    if (!dtype_ok(dtype)) return fail(FTQ_ERR_INVALID, "bad dtype %d", dtype);
    if (n_vec == 0) return FTQ_OK;
    if (!x || !y || n_vec < 0) return fail(FTQ_ERR_INVALID, "bad tensor argument");
    if (!aligned(x, 16) || !aligned(y, 4)) return fail(FTQ_ERR_INVALID, "misaligned tensor");
    ftq::SignBits sg;
    int rc = pack_signs(signs_host, head_dim, &sg);
    if (rc) return rc;
    const float r = rsqrt_dim(head_dim);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned grid = grid_for(n_vec, 32);
#define FTQ_RT(DD)                                                                              \
    switch (dtype) {                                                                            \
        case FTQ_F32:                                                                           \
            ftq::rht_kernel<DD, float><<<grid, 256, 0, st>>>(                                    \
                static_cast<const float*>(x), static_cast<float*>(y), sg, r, inverse, n_vec);   \
            break;                                                                              \
        case FTQ_F16:                                                                           \
            ftq::rht_kernel<DD, __half><<<grid, 256, 0, st>>>(                                   \
                static_cast<const __half*>(x), static_cast<__half*>(y), sg, r, inverse, n_vec); \
            break;                                                                              \
        case FTQ_BF16:                                                                          \
            ftq::rht_kernel<DD, __nv_bfloat16><<<grid, 256, 0, st>>>(                            \
                static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), sg, r,    \
                inverse, n_vec);                                                                \
            break;                                                                              \
    }
    switch (head_dim) {
        case 64: FTQ_RT(64) break;
        case 128: FTQ_RT(128) break;
        case 256: FTQ_RT(256) break;
    }
#undef FTQ_RT
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FTQ_OK : cuda_fail(e, "ftq_rht launch");
}

int ftq_qk_scores(const float* q_rot, const uint8_t* k_codes, const void* k_norms, int norms_dtype,
                  const float* levels_host, float scale, int bits, int B, int Hq, int Hkv,
                  int q_len, int S, int head_dim, float* out, void* stream) {
    if (!dim_ok(head_dim)) return fail(FTQ_ERR_UNSUPPORTED, "head_dim %d (need 64/128/256)", head_dim);
    if (!bits_ok(bits)) return fail(FTQ_ERR_INVALID, "bits must be 2, 3, or 4, got %d", bits);
    if (norms_dtype != FTQ_F16 && norms_dtype != FTQ_F32)
        return fail(FTQ_ERR_INVALID, "norms must be fp16 or fp32");
    if (B < 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv || q_len <= 0 || S < 0)
        return fail(FTQ_ERR_INVALID, "bad shape B=%d Hq=%d Hkv=%d q_len=%d S=%d", B, Hq, Hkv, q_len, S);
    if (B == 0 || S == 0) return FTQ_OK;
    if (!q_rot || !k_codes || !k_norms || !out) return fail(FTQ_ERR_INVALID, "NULL tensor pointer");
    if (!aligned(k_codes, 4)) return fail(FTQ_ERR_INVALID, "k_codes must be 4-byte aligned");
    ftq::Codebook lv;
    int rc = pack_levels(levels_host, bits, &lv);
    if (rc) return rc;
    const int rows = (Hq / Hkv) * q_len;
    const size_t smem = (ftq::kMaxLevels + static_cast<size_t>(rows) * head_dim) * sizeof(float);
    if (smem > 48 * 1024)
        return fail(FTQ_ERR_UNSUPPORTED, "group*q_len*head_dim = %d exceeds the 48 KB query tile",
                    rows * head_dim);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const dim3 grid((S + 63) / 64, B * Hkv);
#define FTQ_QK(DD, BB)                                                                          \
    if (norms_dtype == FTQ_F16)                                                                 \
        ftq::qk_scores_kernel<DD, BB, __half><<<grid, 128, smem, st>>>(                          \
            q_rot, k_codes, static_cast<const __half*>(k_norms), out, lv, scale, Hq, Hkv, q_len, S); \
    else                                                                                        \
        ftq::qk_scores_kernel<DD, BB, float><<<grid, 128, smem, st>>>(                           \
            q_rot, k_codes, static_cast<const float*>(k_norms), out, lv, scale, Hq, Hkv, q_len, S);
#define FTQ_QB(DD)                                                                              \
    switch (bits) {                                                                             \
        case 2: FTQ_QK(DD, 2) break;                                                            \
        case 3: FTQ_QK(DD, 3) break;                                                            \
        case 4: FTQ_QK(DD, 4) break;                                                            \
    }
    switch (head_dim) {
        case 64: FTQ_QB(64) break;
        case 128: FTQ_QB(128) break;
        case 256: FTQ_QB(256) break;
    }
#undef FTQ_QB
#undef FTQ_QK
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FTQ_OK : cuda_fail(e, "ftq_qk_scores launch");
}

// The tail of a decode workspace holds the counters of the tensor-core kernels: a 256-byte header
// (work-item counter, count of finished CTAs, the 64-bit epoch word) and, from byte 256 on, one
// counter per (layer, sequence, KV head) unit for the in-kernel split-KV merge.  The
// barrier-synchronised kernel's launcher zeroes the header with a memset node; the streaming
// kernel clears the tail itself under a per-launch epoch (see AttnParams), so one call is one
// node in the stream and needs nothing from the call before it.
static unsigned long long next_epoch() {
    static std::atomic<unsigned long long> counter{[] {
        std::random_device rd;
        return (static_cast<unsigned long long>(rd()) << 32) | 1ull;
    }()};
    unsigned long long e = counter.fetch_add(1, std::memory_order_relaxed);
    return e ? e : counter.fetch_add(1, std::memory_order_relaxed);
}

static size_t counter_bytes(int B, int Hkv, int n_layers) {
    const size_t units = static_cast<size_t>(n_layers > 0 ? n_layers : 0) * (B > 0 ? B : 0) *
                         (Hkv > 0 ? Hkv : 0);
    return (256 + units * sizeof(int) + 255) / 256 * 256;
}

size_t ftq_decode_workspace_bytes(int B, int Hq, int Hkv, int head_dim, int max_seq_len,
                                  int n_layers) {
    if (!dim_ok(head_dim) || B <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv || n_layers <= 0) return 0;
    // the larger of the two paths' needs, so one buffer serves whichever kernel runs
    const ChunkPlan a = plan_chunks(B, Hq, Hkv, head_dim, max_seq_len, n_layers);
    const ChunkPlan m1 = plan_chunks_mma(B, Hkv, max_seq_len, n_layers, 1);
    const ChunkPlan m2 = plan_chunks_mma(B, Hkv, max_seq_len, n_layers, 2);
    const ChunkPlan m3 = plan_chunks_stream(B, Hkv, max_seq_len, n_layers, 1);
    const ChunkPlan m4 = plan_chunks_stream(B, Hkv, max_seq_len, n_layers, 2);
    size_t n = partial_bytes(a, B, Hq, head_dim, n_layers);
    const size_t n3 = partial_bytes(m3, B, Hq, head_dim, n_layers);
    const size_t n4 = partial_bytes(m4, B, Hq, head_dim, n_layers);
    if (n3 > n) n = n3;
    if (n4 > n) n = n4;
    const size_t n1 = partial_bytes(m1, B, Hq, head_dim, n_layers);
    const size_t n2 = partial_bytes(m2, B, Hq, head_dim, n_layers);
    if (n1 > n) n = n1;
    if (n2 > n) n = n2;
    return n + counter_bytes(B, Hkv, n_layers);
}

static int check_attn_common(int B, int Hq, int Hkv, int head_dim, int bits_k, int bits_v,
                             int q_dtype, int out_dtype) {
    if (!dim_ok(head_dim)) return fail(FTQ_ERR_UNSUPPORTED, "head_dim %d (need 64/128/256)", head_dim);
    if (!bits_ok(bits_k) || !bits_ok(bits_v))
        return fail(FTQ_ERR_INVALID, "bits must be 2, 3, or 4, got K=%d V=%d", bits_k, bits_v);
    if (!dtype_ok(q_dtype) || !dtype_ok(out_dtype)) return fail(FTQ_ERR_INVALID, "bad dtype");
    if (B < 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv)
        return fail(FTQ_ERR_INVALID, "bad shape B=%d Hq=%d Hkv=%d", B, Hq, Hkv);
    return FTQ_OK;
}

int ftq_flash_decode(const void* q, int q_dtype, int q_is_rotated, const uint8_t* k_codes,
                     const uint16_t* k_norms, const uint8_t* v_codes, const uint16_t* v_norms,
                     const float* levels_k_host, const float* levels_v_host,
                     const float* signs_host, float scale, int bits_k, int bits_v,
                     const int32_t* seq_lens, int B, int Hq, int Hkv, int S, int head_dim,
                     void* out, int out_dtype, void* workspace, size_t workspace_bytes,
                     void* stream) {
    int rc = check_attn_common(B, Hq, Hkv, head_dim, bits_k, bits_v, q_dtype, out_dtype);
    if (rc) return rc;
    if (S < 0) return fail(FTQ_ERR_INVALID, "S < 0");
    if (B == 0) return FTQ_OK;
    if (!q || !out) return fail(FTQ_ERR_INVALID, "NULL q / out");
    if (S > 0 && (!k_codes || !k_norms || !v_codes || !v_norms))
        return fail(FTQ_ERR_INVALID, "NULL K/V tensor");
    if (!aligned(q, 16) || !aligned(out, 4)) return fail(FTQ_ERR_INVALID, "q must be 16-byte aligned");
    if (!aligned(k_codes, 4) || !aligned(v_codes, 4) || !aligned(k_norms, 2) || !aligned(v_norms, 2))
        return fail(FTQ_ERR_INVALID, "misaligned K/V tensor");
    const ChunkPlan pl = plan_chunks(B, Hq, Hkv, head_dim, S, 1);
    const size_t need = partial_bytes(pl, B, Hq, head_dim, 1);
    if (!workspace || workspace_bytes < need)
        return fail(FTQ_ERR_WORKSPACE, "workspace needs %zu bytes, got %zu", need, workspace_bytes);
    if (!aligned(workspace, 16)) return fail(FTQ_ERR_WORKSPACE, "workspace must be 16-byte aligned");
    ftq::AttnParams p{};
    rc = pack_levels(levels_k_host, bits_k, &p.lk);
    if (rc) return rc;
    rc = pack_levels(levels_v_host, bits_v, &p.lv);
    if (rc) return rc;
    rc = pack_signs(signs_host, head_dim, &p.signs);
    if (rc) return rc;
    const int pdk = ftq::packed_dim(head_dim, bits_k), pdv = ftq::packed_dim(head_dim, bits_v);
    p.q = q;
    p.k_codes = k_codes; p.k_norms = k_norms; p.v_codes = v_codes; p.v_norms = v_norms;
    p.S = S; p.seq_lens = seq_lens; p.B = B; p.Hq = Hq; p.Hkv = Hkv;
    p.scale = scale; p.q_is_rotated = q_is_rotated; p.q_dtype = q_dtype;
    p.cp16 = aligned(k_codes, 16) && aligned(v_codes, 16) &&
             (static_cast<int64_t>(S) * pdk) % 16 == 0 && (static_cast<int64_t>(S) * pdv) % 16 == 0;
    p.chunk_tokens = pl.chunk_tokens; p.n_chunks = pl.n_chunks; p.n_hpass = pl.n_hpass;
    p.partials = static_cast<float*>(workspace);
    p.rsqrt_d = rsqrt_dim(head_dim);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = dispatch_split(head_dim, bits_k, bits_v, false, p, B, st);
    if (e != cudaSuccess) return cuda_fail(e, "ftq_flash_decode split launch");
    e = dispatch_merge(head_dim, out_dtype, p.partials, out, seq_lens, S, B, Hq, Hkv, pl,
                       ftq::SplitPlan{}, static_cast<int64_t>(B) * Hq, p.signs, st);
    return e == cudaSuccess ? FTQ_OK : cuda_fail(e, "ftq_flash_decode merge launch");
}

int ftq_paged_store(const void* key, const void* value, int dtype, int64_t n_tokens, int Hkv,
                    int head_dim, int64_t token_stride, int64_t head_stride, int bits_k,
                    int bits_v, const float* signs_host, const float* boundaries_k_host,
                    const float* boundaries_v_host, uint8_t* pool, int64_t num_blocks,
                    const int64_t* slot_mapping, int n_layers, int64_t kv_layer_stride,
                    int64_t pool_layer_stride, void* stream) {
    if (!dim_ok(head_dim)) return fail(FTQ_ERR_UNSUPPORTED, "head_dim %d (need 64/128/256)", head_dim);
    if (!bits_ok(bits_k) || !bits_ok(bits_v))
        return fail(FTQ_ERR_INVALID, "bits must be 2, 3, or 4, got K=%d V=%d", bits_k, bits_v);
    if (!dtype_ok(dtype)) return fail(FTQ_ERR_INVALID, "bad dtype %d", dtype);
    if (n_tokens * Hkv >= (1ll << 31) || num_blocks * Hkv >= (1ll << 31))
        return fail(FTQ_ERR_INVALID, "n_tokens * Hkv and num_blocks * Hkv must be below 2^31");
    if (n_tokens < 0 || Hkv <= 0 || n_layers <= 0 || num_blocks < 0)
        return fail(FTQ_ERR_INVALID, "bad shape");
    if (n_tokens == 0) return FTQ_OK;
    if (!key || !value || !pool || !slot_mapping) return fail(FTQ_ERR_INVALID, "NULL tensor pointer");
    const size_t es = dtype_size(dtype);
    if (!aligned(key, 16) || !aligned(value, 16) || (token_stride * es) % 16 ||
        (head_stride * es) % 16 || (kv_layer_stride * es) % 16)
        return fail(FTQ_ERR_INVALID, "key/value rows must be 16-byte aligned");
    if (!aligned(pool, 16) || pool_layer_stride % 16)
        return fail(FTQ_ERR_INVALID, "pool must be 16-byte aligned");
    const int pdk = ftq::packed_dim(head_dim, bits_k), pdv = ftq::packed_dim(head_dim, bits_v);
    const int64_t page = ftq_page_bytes(head_dim, bits_k, bits_v);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    for (int which = 0; which < 2; which++) {
        ftq::EncodeTables tab;
        int rc = make_encode_tables(head_dim, which ? bits_v : bits_k, signs_host,
                                    which ? boundaries_v_host : boundaries_k_host, &tab);
        if (rc) return rc;
        ftq::EncodeSource src{which ? value : key, Hkv, token_stride, head_stride, kv_layer_stride};
        ftq::EncodeSink sink{};
        sink.mode = ftq::kSinkPaged;
        sink.codes = pool;
        sink.slot_mapping = slot_mapping;
        sink.Hkv = Hkv;
        sink.page_bytes = page;
        sink.slot_limit = num_blocks * FTQ_PAGE_TOKENS;
        sink.codes_off = which ? FTQ_PAGE_TOKENS * pdk + 2 * FTQ_PAGE_TOKENS : 0;
        sink.norms_off = which ? FTQ_PAGE_TOKENS * (pdk + pdv) + 2 * FTQ_PAGE_TOKENS
                               : FTQ_PAGE_TOKENS * pdk;
        sink.layer_stride = pool_layer_stride;
        sink.swap_halves = which;  // V rows only (see the page layout in ftq_b200.h)
        cudaError_t e = dispatch_encode(head_dim, which ? bits_v : bits_k, dtype, src, sink, tab,
                                        n_tokens * Hkv, n_layers, st);
        if (e != cudaSuccess) return cuda_fail(e, "ftq_paged_store launch");
    }
    return FTQ_OK;
}

int ftq_paged_decode_attn(const void* q, int q_dtype, void* out, int out_dtype,
                          const uint8_t* pool, int64_t num_blocks, int64_t pool_layer_stride,
                          int n_layers, const int32_t* block_table, int max_blocks,
                          const int32_t* seq_lens, int max_seq_len, int B, int Hq, int Hkv,
                          int head_dim, int bits_k, int bits_v, const float* levels_k_host,
                          const float* levels_v_host, const float* signs_host, float scale,
                          void* workspace, size_t workspace_bytes, void* stream) {
    int rc = check_attn_common(B, Hq, Hkv, head_dim, bits_k, bits_v, q_dtype, out_dtype);
    if (rc) return rc;
    if (n_layers <= 0 || max_blocks < 0 || max_seq_len < 0 || num_blocks < 0)
        return fail(FTQ_ERR_INVALID, "bad shape");
    if (B == 0) return FTQ_OK;
    if (!q || !out || !pool || !block_table || !seq_lens)
        return fail(FTQ_ERR_INVALID, "NULL tensor pointer");
    if (static_cast<int64_t>(max_blocks) * FTQ_PAGE_TOKENS < max_seq_len)
        return fail(FTQ_ERR_INVALID, "block_table too narrow: %d blocks < max_seq_len %d",
                    max_blocks, max_seq_len);
    if (!aligned(q, 16) || !aligned(out, 4) || !aligned(pool, 16) || pool_layer_stride % 16)
        return fail(FTQ_ERR_INVALID, "q and pool must be 16-byte aligned");
    // 16-bit queries with a GQA group of at most 8 take the tensor-core kernel; fp32 queries
    // (and larger groups) take the fp32 kernel.
    const bool mma = use_mma_path(Hq, Hkv, q_dtype);
    // one CTA per SM (16 warps) when a 4-bit byte table is in use, else two (8 warps each)
    const int mma_ctas = (bits_k == 4 || bits_v == 4) ? 1 : 2;
    const int stream_ctas = mma ? attn_mma_stream_ctas(head_dim, bits_k, bits_v, Hq / Hkv) : 0;
    const bool streams = stream_ctas > 0;
    const ChunkPlan pl = streams ? plan_chunks_stream(B, Hkv, max_seq_len, n_layers, stream_ctas)
                         : mma   ? plan_chunks_mma(B, Hkv, max_seq_len, n_layers, mma_ctas)
                                 : plan_chunks(B, Hq, Hkv, head_dim, max_seq_len, n_layers);
    const size_t need = ftq_decode_workspace_bytes(B, Hq, Hkv, head_dim, max_seq_len, n_layers);
    if (!workspace || workspace_bytes < need)
        return fail(FTQ_ERR_WORKSPACE, "workspace needs %zu bytes, got %zu", need, workspace_bytes);
    if (!aligned(workspace, 16)) return fail(FTQ_ERR_WORKSPACE, "workspace must be 16-byte aligned");
    ftq::AttnParams p{};
    rc = pack_levels(levels_k_host, bits_k, &p.lk);
    if (rc) return rc;
    rc = pack_levels(levels_v_host, bits_v, &p.lv);
    if (rc) return rc;
    rc = pack_signs(signs_host, head_dim, &p.signs);
    if (rc) return rc;
    p.q = q;
    p.num_blocks = num_blocks;
    p.pool = pool; p.pool_layer_stride = pool_layer_stride;
    p.block_table = block_table; p.max_blocks = max_blocks;
    p.S = 0; p.seq_lens = seq_lens; p.B = B; p.Hq = Hq; p.Hkv = Hkv;
    p.scale = scale; p.q_is_rotated = 0; p.q_dtype = q_dtype; p.cp16 = 1;
    p.chunk_tokens = pl.chunk_tokens; p.n_chunks = pl.n_chunks; p.n_hpass = pl.n_hpass;
    p.partials = static_cast<float*>(workspace);
    p.rsqrt_d = rsqrt_dim(head_dim);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    {
        const size_t tail = counter_bytes(B, Hkv, n_layers);
        p.work_counter = reinterpret_cast<int*>(static_cast<uint8_t*>(workspace) + need - tail);
    }
    if (mma) {
        const float vs = choose_v_scale(levels_v_host, bits_v, head_dim);
        for (int i = 0; i < (1 << bits_v); i++) p.lv_scaled.v[i] = levels_v_host[i] * vs;
        p.inv_v_scale = 1.0f / vs;
        // K centroids scaled for the smallest fp16 rounding error, undone through the softmax scale
        const float ks = choose_k_scale(levels_k_host, bits_k, head_dim);
        for (int i = 0; i < (1 << bits_k); i++) p.lk.v[i] = levels_k_host[i] * ks;
        p.scale = scale / ks;
        // K and V can share one table only when the scaled V levels equal the K levels
        const bool shared_lut = bits_k == bits_v &&
            memcmp(p.lk.v, p.lv_scaled.v, sizeof(float) << bits_k) == 0;
        p.unit_counter = p.work_counter + 64;
        p.out = out;
        p.out_dtype = out_dtype;
        p.num_blocks = num_blocks;
        p.div_chunks = ftq::make_fastdiv(static_cast<uint32_t>(p.n_chunks));
        p.div_hkv = ftq::make_fastdiv(static_cast<uint32_t>(Hkv));
        p.div_b = ftq::make_fastdiv(static_cast<uint32_t>(B));
        p.n_units = n_layers * B * Hkv;
        p.epoch = next_epoch();
        p.split = make_split(pl, p.n_units, true);
        bool merged = false;
        e = dispatch_mma(head_dim, bits_k, bits_v, shared_lut, p, n_layers * B, st, &merged);
        if (e != cudaSuccess) return cuda_fail(e, "ftq_paged_decode_attn launch");
        if (merged) return FTQ_OK;  // the streaming kernel finishes the merge itself
    } else {
        e = cudaMemsetAsync(p.work_counter, 0, 256, st);   // the status word
        if (e != cudaSuccess) return cuda_fail(e, "ftq_paged_decode_attn status reset");
        e = dispatch_split(head_dim, bits_k, bits_v, true, p, n_layers * B, st);
    }
    if (e != cudaSuccess) return cuda_fail(e, "ftq_paged_decode_attn split launch");
    e = dispatch_merge(head_dim, out_dtype, p.partials, out, seq_lens, 0, B, Hq, Hkv, pl,
                       p.split, static_cast<int64_t>(n_layers) * B * Hq, p.signs, st);
    return e == cudaSuccess ? FTQ_OK : cuda_fail(e, "ftq_paged_decode_attn merge launch");
}

int ftq_v0_store(const void* key, const void* value, int dtype, int64_t n_tokens, int Hkv,
                 int head_dim, int64_t token_stride, int64_t head_stride, int bits_k, int bits_v,
                 const float* signs_host, const float* boundaries_k_host,
                 const float* boundaries_v_host, uint8_t* kv_cache, int64_t num_blocks,
                 int block_size, int elem_size, const int64_t* slot_mapping, void* stream) {
    if (!dim_ok(head_dim)) return fail(FTQ_ERR_UNSUPPORTED, "head_dim %d (need 64/128/256)", head_dim);
    if (!bits_ok(bits_k) || !bits_ok(bits_v))
        return fail(FTQ_ERR_INVALID, "bits must be 2, 3, or 4, got K=%d V=%d", bits_k, bits_v);
    if (!dtype_ok(dtype)) return fail(FTQ_ERR_INVALID, "bad dtype %d", dtype);
    if (n_tokens * Hkv >= (1ll << 31))
        return fail(FTQ_ERR_INVALID, "n_tokens * Hkv must be below 2^31 per call");
    if (n_tokens < 0 || Hkv <= 0 || block_size <= 0 || num_blocks < 0)
        return fail(FTQ_ERR_INVALID, "bad shape");
    const int pdk = ftq::packed_dim(head_dim, bits_k), pdv = ftq::packed_dim(head_dim, bits_v);
    if (elem_size < (pdk > pdv ? pdk : pdv) + 4 || elem_size % 4)
        return fail(FTQ_ERR_INVALID, "elem_size %d too small for packed_dim + 4", elem_size);
    if (n_tokens == 0) return FTQ_OK;
    if (!key || !value || !kv_cache || !slot_mapping) return fail(FTQ_ERR_INVALID, "NULL tensor pointer");
    const size_t es = dtype_size(dtype);
    if (!aligned(key, 16) || !aligned(value, 16) || (token_stride * es) % 16 || (head_stride * es) % 16)
        return fail(FTQ_ERR_INVALID, "key/value rows must be 16-byte aligned");
    if (!aligned(kv_cache, 4)) return fail(FTQ_ERR_INVALID, "kv_cache must be 4-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    for (int which = 0; which < 2; which++) {
        ftq::EncodeTables tab;
        int rc = make_encode_tables(head_dim, which ? bits_v : bits_k, signs_host,
                                    which ? boundaries_v_host : boundaries_k_host, &tab);
        if (rc) return rc;
        ftq::EncodeSource src{which ? value : key, Hkv, token_stride, head_stride, 0};
        ftq::EncodeSink sink{};
        sink.mode = ftq::kSinkV0;
        sink.codes = kv_cache;
        sink.slot_mapping = slot_mapping;
        sink.Hkv = Hkv;
        sink.block_size = block_size;
        sink.slot_limit = num_blocks * block_size;
        sink.elem_size = elem_size;
        sink.plane_off = static_cast<int64_t>(which) * num_blocks * block_size * Hkv * elem_size;
        cudaError_t e = dispatch_encode(head_dim, which ? bits_v : bits_k, dtype, src, sink, tab,
                                        n_tokens * Hkv, 1, st);
        if (e != cudaSuccess) return cuda_fail(e, "ftq_v0_store launch");
    }
    return FTQ_OK;
}

int ftq_v0_gather(const uint8_t* kv_cache, int64_t num_blocks, int block_size, int Hkv,
                  int elem_size, int kv_type, int packed_dim, const int32_t* block_tables,
                  int max_blocks, const int32_t* seq_lens, int B, int max_seq_len,
                  uint8_t* out_codes, float* out_norms, void* stream) {
    if (B < 0 || Hkv <= 0 || block_size <= 0 || max_seq_len < 0 || packed_dim <= 0 ||
        packed_dim % 4 || elem_size < packed_dim + 4 || elem_size % 4 || (kv_type != 0 && kv_type != 1))
        return fail(FTQ_ERR_INVALID, "bad shape");
    if (B == 0 || max_seq_len == 0) return FTQ_OK;
    if (!kv_cache || !block_tables || !seq_lens || !out_codes || !out_norms)
        return fail(FTQ_ERR_INVALID, "NULL tensor pointer");
    if (!aligned(kv_cache, 4) || !aligned(out_codes, 4))
        return fail(FTQ_ERR_INVALID, "kv_cache / out_codes must be 4-byte aligned");
    const int64_t total = static_cast<int64_t>(B) * Hkv * max_seq_len * (packed_dim / 4 + 1);
    const int64_t want = (total + 255) / 256;
    const int64_t cap = static_cast<int64_t>(ftq::sm_count()) * 16;
    const unsigned grid = static_cast<unsigned>(want < cap ? want : cap);
    v0_gather_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        kv_cache, num_blocks, block_size, Hkv, elem_size, kv_type, packed_dim, block_tables,
        max_blocks, seq_lens, B, max_seq_len, out_codes, out_norms);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FTQ_OK : cuda_fail(e, "ftq_v0_gather launch");
}

}  // extern "C"

// --------------------------------------------------------------------------
// Paged decode attention without a caller workspace.
//
// Some callers have no memory to give and cannot get any: an inference engine
// that has already handed (nearly) all of the device to its own KV block
// manager, a plugin that is entered in a context where cudaMalloc is not
// allowed or would stall the device (it synchronises), or a host that simply
// forbids allocation after start-up.  For them the split-KV partials live in a
// fixed array inside the library image instead.  The price: the array occupies
// FTQ_STATIC_SCRATCH_BYTES on every GPU that loads the library, for the life
// of the process, and it caps the problem size.
static __device__ __align__(256) unsigned char g_static_scratch[FTQ_STATIC_SCRATCH_BYTES];

namespace {
std::mutex g_static_mu;
void* g_static_addr[64] = {nullptr};

// In host code `g_static_scratch` is only a handle for the symbol; the device
// address has to be asked for, once per device, with that device current.
int static_scratch_address(void** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev < 0 || dev >= 64) return fail(FTQ_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!g_static_addr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(static scratch)");
        if (!p) return fail(FTQ_ERR_CUDA, "static scratch has no device address");
        g_static_addr[dev] = p;
    }
    *out = g_static_addr[dev];
    return FTQ_OK;
}
}  // namespace

extern "C" int ftq_paged_decode_attn_static(
    const void* q, int q_dtype, void* out, int out_dtype, const uint8_t* pool, int64_t num_blocks,
    int64_t pool_layer_stride, int n_layers, const int32_t* block_table, int max_blocks,
    const int32_t* seq_lens, int max_seq_len, int B, int Hq, int Hkv, int head_dim, int bits_k,
    int bits_v, const float* levels_k_host, const float* levels_v_host, const float* signs_host,
    float scale, void* stream) {
    // Argument errors first (the shared path reports the rest), then the size limit.
    const int bad = check_attn_common(B, Hq, Hkv, head_dim, bits_k, bits_v, q_dtype, out_dtype);
    if (bad) return bad;
    const size_t need = ftq_decode_workspace_bytes(B, Hq, Hkv, head_dim, max_seq_len, n_layers);
    if (need > static_cast<size_t>(FTQ_STATIC_SCRATCH_BYTES))
        return fail(FTQ_ERR_WORKSPACE,
                    "this batch needs %zu bytes of split-KV scratch but the built-in scratch holds "
                    "%zu; call ftq_paged_decode_attn with your own workspace, or pass fewer "
                    "sequences / layers per call",
                    need, static_cast<size_t>(FTQ_STATIC_SCRATCH_BYTES));
    void* scratch = nullptr;
    const int rc = static_scratch_address(&scratch);
    if (rc) return rc;
    return ftq_paged_decode_attn(q, q_dtype, out, out_dtype, pool, num_blocks, pool_layer_stride,
                                 n_layers, block_table, max_blocks, seq_lens, max_seq_len, B, Hq,
                                 Hkv, head_dim, bits_k, bits_v, levels_k_host, levels_v_host,
                                 signs_host, scale, scratch, FTQ_STATIC_SCRATCH_BYTES, stream);
}

extern "C" int ftq_paged_decode_status(const void* workspace, int B, int Hq, int Hkv, int head_dim,
                                       int max_seq_len, int n_layers, void* stream,
                                       int* status_bits) {
    const size_t need = ftq_decode_workspace_bytes(B, Hq, Hkv, head_dim, max_seq_len, n_layers);
    if (need == 0) return fail(FTQ_ERR_INVALID, "bad shape");
    const void* base = workspace;
    if (!base) {
        if (need > static_cast<size_t>(FTQ_STATIC_SCRATCH_BYTES))
            return fail(FTQ_ERR_WORKSPACE, "no such call can have used the built-in scratch");
        void* scratch = nullptr;
        const int rc = static_scratch_address(&scratch);
        if (rc) return rc;
        base = scratch;
    }
    const uint8_t* word = static_cast<const uint8_t*>(base) + need - counter_bytes(B, Hkv, n_layers) +
                          ftq::kStatusWord * sizeof(int);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int bits = 0;
    cudaError_t e = cudaMemcpyAsync(&bits, word, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return cuda_fail(e, "ftq_paged_decode_status");
    if (status_bits) *status_bits = bits;
    if (bits == 0) return FTQ_OK;
    return fail(FTQ_ERR_DEVICE, "the last decode call on this workspace reported%s%s",
                (bits & FTQ_STATUS_BAD_BLOCK_ID) ? " a block id outside the pool" : "",
                (bits & FTQ_STATUS_WAIT_EXPIRED) ? " a wait that ran out" : "");
}

// ------------------------------------------------------------------ vLLM-v1 slot format

namespace {
// key_bits 8 = FP8 (e4m3) keys, as in vLLM's stock TurboQuantConfig
// key_bits: 1..4 = Lloyd-Max codes, 8 = FP8, FTQ_TQ_KEY_BITS_MSE8 = 8-bit Lloyd-Max codes
bool tq_bits_ok(int kb, int vb) {
    return ((kb >= 1 && kb <= 4) || kb == 8 || kb == FTQ_TQ_KEY_BITS_MSE8) && ((vb >= 1 && vb <= 4) || vb == 8);
}
int tq_key_bytes(int d, int kb) {
    return kb == 8 ? d : (kb == FTQ_TQ_KEY_BITS_MSE8 ? d + 2 : d * kb / 8 + 2);
}
static_assert(FTQ_TQ_KEY_BITS_MSE8 == ftq::kTqKeyBitsMse8, "header and kernels agree on the marker");
// strictly ascending table of n floats -> the kernels' 256-entry parameter block
int pack_table256(const float* host, int n, bool ascending_strictly, ftq::TqTable256* t) {
    for (int i = 0; i < 256; i++) t->v[i] = i < n ? host[i] : FLT_MAX;
    for (int i = 1; i < n; i++)
        if (ascending_strictly ? !(host[i] > host[i - 1]) : !(host[i] >= host[i - 1]))
            return fail(FTQ_ERR_INVALID, "the 8-bit key table must be ascending");
    return FTQ_OK;
}
bool even(int64_t v) { return (v & 1) == 0; }
}  // namespace

extern "C" int ftq_tq_slot_bytes(int head_dim, int key_bits, int value_bits) {
    if (!dim_ok(head_dim) || !tq_bits_ok(key_bits, value_bits)) return -1;
    const int s = tq_key_bytes(head_dim, key_bits) + ftq::tq_value_bytes(head_dim, value_bits) + 4;
    return s + (s & 1);
}

extern "C" int ftq_tq_store(const void* key, const void* value, int dtype, int64_t n_tokens, int Hkv,
                            int head_dim, int64_t token_stride, int64_t head_stride, int key_bits,
                            int value_bits, int rotate_values, int value_lloyd_max,
                            const float* midpoints_host, uint8_t* kv_cache,
                            int64_t stride_block, int64_t stride_pos, int64_t stride_head,
                            int block_size, const int64_t* slot_mapping, void* stream) {
    return ftq_tq_store_layers(key, value, dtype, n_tokens, Hkv, head_dim, token_stride, head_stride,
                               key_bits, value_bits, rotate_values, value_lloyd_max, midpoints_host,
                               kv_cache, stride_block, stride_pos, stride_head, block_size,
                               slot_mapping, 1, 0, 0, 0, stream);
}

extern "C" int ftq_tq_store_layers(const void* key, const void* value, int dtype, int64_t n_tokens,
                                   int Hkv, int head_dim, int64_t token_stride, int64_t head_stride,
                                   int key_bits, int value_bits, int rotate_values,
                                   int value_lloyd_max, const float* midpoints_host,
                                   uint8_t* kv_cache, int64_t stride_block, int64_t stride_pos,
                                   int64_t stride_head, int block_size,
                                   const int64_t* slot_mapping, int n_layers,
                                   int64_t kv_layer_stride, int64_t cache_layer_stride,
                                   int64_t num_blocks, void* stream) {
    if (n_layers <= 0 || n_layers > 65535 || !even(cache_layer_stride) || num_blocks < 0)
        return fail(FTQ_ERR_INVALID, "bad n_layers / cache_layer_stride / num_blocks");
    if (!dim_ok(head_dim)) return fail(FTQ_ERR_UNSUPPORTED, "head_dim %d (need 64/128/256)", head_dim);
    if (!tq_bits_ok(key_bits, value_bits))
        return fail(FTQ_ERR_UNSUPPORTED, "key_bits %d / value_bits %d (need 1..4, 8 = FP8 or FTQ_TQ_KEY_BITS_MSE8 / 1,2,3,4,8)", key_bits,
                    value_bits);
    if (!dtype_ok(dtype)) return fail(FTQ_ERR_INVALID, "bad dtype %d", dtype);
    if (rotate_values && value_bits == 8)
        return fail(FTQ_ERR_UNSUPPORTED, "rotate_values with 8-bit values: rotate them before the call");
    if (n_tokens < 0 || Hkv <= 0 || block_size <= 0) return fail(FTQ_ERR_INVALID, "bad shape");
    if (n_tokens * Hkv >= (1ll << 31)) return fail(FTQ_ERR_INVALID, "n_tokens * Hkv must be below 2^31");
    if (n_tokens == 0) return FTQ_OK;
    const bool key_fp8 = key_bits == 8;  // no codebook: midpoints_host may be NULL
    const bool key_mse8 = key_bits == FTQ_TQ_KEY_BITS_MSE8;  // midpoints_host: 255 entries
    if ((key_fp8 || key_mse8) && value_lloyd_max && value_bits == 4)
        return fail(FTQ_ERR_UNSUPPORTED, "Lloyd-Max value codes need a 4-bit key codebook");
    if (!key || !value || !kv_cache || !slot_mapping || (!key_fp8 && !midpoints_host))
        return fail(FTQ_ERR_INVALID, "NULL pointer argument");
    const int64_t es = static_cast<int64_t>(dtype_size(dtype));
    if (!aligned(key, 16) || !aligned(value, 16) || (token_stride * es) % 16 || (head_stride * es) % 16 ||
        (kv_layer_stride * es) % 16)
        return fail(FTQ_ERR_INVALID, "key/value rows must be 16-byte aligned");
    if (!aligned(kv_cache, 2) || !even(stride_block) || !even(stride_pos) || !even(stride_head))
        return fail(FTQ_ERR_INVALID, "kv_cache base and strides must be even");
    if (stride_head < ftq_tq_slot_bytes(head_dim, key_bits, value_bits) - 1)
        return fail(FTQ_ERR_INVALID, "stride_head smaller than the slot");
    ftq::TqStoreParams p{};
    p.kv_layer_stride = kv_layer_stride;
    p.cache_layer_stride = cache_layer_stride;
    // (num_blocks = 0: the cache's extent is not known, only negative slots are skipped)
    p.slot_limit = num_blocks > 0 ? num_blocks * block_size : INT64_MAX;
    p.key = key;
    p.value = value;
    p.token_stride = token_stride;
    p.head_stride = head_stride;
    p.Hkv = Hkv;
    p.div_hkv = ftq::make_fastdiv(static_cast<uint32_t>(Hkv));
    p.kv_cache = kv_cache;
    p.stride_block = stride_block;
    p.stride_pos = stride_pos;
    p.stride_head = stride_head;
    p.block_size = block_size;
    p.div_block = ftq::make_fastdiv(static_cast<uint32_t>(block_size));
    p.slot_mapping = slot_mapping;
    const int nmid = (key_fp8 || key_mse8) ? 0 : (1 << key_bits) - 1;
    for (int i = 0; i < ftq::kTqMaxMid; i++) p.midpoints[i] = i < nmid ? midpoints_host[i] : FLT_MAX;
    for (int i = 1; i < nmid; i++)
        if (!(midpoints_host[i] > midpoints_host[i - 1]))
            return fail(FTQ_ERR_INVALID, "midpoints must be strictly ascending");
    ftq::TqTable256 mid8;
    if (key_mse8) {
        const int rc = pack_table256(midpoints_host, 255, true, &mid8);
        if (rc) return rc;
    }
    const ftq::TqTable256* t8 = key_mse8 ? &mid8 : nullptr;
    const int kb = key_mse8 ? 8 : key_bits;
    p.rsqrt_d = 1.0f / sqrtf(static_cast<float>(head_dim));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t n_vec = n_tokens * Hkv;
    // (as in the reference, the Lloyd-Max flag only changes 4-bit values)
    const int vmode = (rotate_values ? ftq::kTqRotateValues : 0) |
                      (value_lloyd_max && value_bits == 4 ? ftq::kTqLloydMaxValues : 0) |
                      (n_layers << 8);
    cudaError_t e = cudaErrorInvalidValue;
    switch (head_dim) {
        case 64: e = ftq::launch_tq_store_d64(kb, value_bits, dtype, p, vmode, n_vec, t8, st); break;
        case 128: e = ftq::launch_tq_store_d128(kb, value_bits, dtype, p, vmode, n_vec, t8, st); break;
        case 256: e = ftq::launch_tq_store_d256(kb, value_bits, dtype, p, vmode, n_vec, t8, st); break;
    }
    return e == cudaSuccess ? FTQ_OK : cuda_fail(e, "tq_store launch");
}

extern "C" int ftq_tq_decode(const void* q, int q_dtype, int B, int Hq, int Hkv, int head_dim,
                             const uint8_t* kv_cache, int64_t stride_block, int64_t stride_pos,
                             int64_t stride_head, int block_size, const int32_t* block_table,
                             int max_blocks, const int32_t* seq_lens, const int32_t* kv_start_offset,
                             int key_bits, int value_bits, int norm_correction, int rotate_output,
                             int value_lloyd_max, const float* centroids_host, float scale,
                             int num_kv_splits,
                             float* mid_o, void* out, int out_dtype, float* lse,
                             const void* prefix_out, int prefix_dtype, const float* prefix_lse,
                             void* stream) {
    return ftq_tq_decode_layers(q, q_dtype, B, Hq, Hkv, head_dim, kv_cache, stride_block, stride_pos,
                                stride_head, block_size, block_table, max_blocks, seq_lens,
                                kv_start_offset, key_bits, value_bits, norm_correction, rotate_output,
                                value_lloyd_max, centroids_host, scale, num_kv_splits, mid_o, out,
                                out_dtype, lse, prefix_out, prefix_dtype, prefix_lse, 1, 0, 0, stream);
}

extern "C" int ftq_tq_decode_layers(const void* q, int q_dtype, int B, int Hq, int Hkv, int head_dim,
                                    const uint8_t* kv_cache, int64_t stride_block, int64_t stride_pos,
                                    int64_t stride_head, int block_size, const int32_t* block_table,
                                    int max_blocks, const int32_t* seq_lens,
                                    const int32_t* kv_start_offset, int key_bits, int value_bits,
                                    int norm_correction, int rotate_output, int value_lloyd_max,
                                    const float* centroids_host, float scale, int num_kv_splits,
                                    float* mid_o, void* out, int out_dtype, float* lse,
                                    const void* prefix_out, int prefix_dtype, const float* prefix_lse,
                                    int n_layers, int64_t cache_layer_stride, int64_t num_blocks,
                                    void* stream) {
    if (n_layers <= 0 || !even(cache_layer_stride) || num_blocks < 0)
        return fail(FTQ_ERR_INVALID, "bad n_layers / cache_layer_stride / num_blocks");
    const int B_seq = B;
    if (static_cast<int64_t>(B) * n_layers > 65535)
        return fail(FTQ_ERR_INVALID, "B * n_layers must be at most 65535 per call");
    B = B * n_layers;   // rows of q / mid_o / out
    if (!dim_ok(head_dim)) return fail(FTQ_ERR_UNSUPPORTED, "head_dim %d (need 64/128/256)", head_dim);
    if (!tq_bits_ok(key_bits, value_bits))
        return fail(FTQ_ERR_UNSUPPORTED, "key_bits %d / value_bits %d (need 1..4, 8 = FP8 or FTQ_TQ_KEY_BITS_MSE8 / 1,2,3,4,8)", key_bits,
                    value_bits);
    if (!dtype_ok(q_dtype) || !dtype_ok(out_dtype)) return fail(FTQ_ERR_INVALID, "bad dtype");
    if ((prefix_out != nullptr) != (prefix_lse != nullptr))
        return fail(FTQ_ERR_INVALID, "prefix_out and prefix_lse go together");
    if (prefix_out && (!dtype_ok(prefix_dtype) || !aligned(prefix_out, 4) || !aligned(prefix_lse, 4)))
        return fail(FTQ_ERR_INVALID, "bad prefix dtype or alignment");
    if (B < 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv || block_size <= 0 || max_blocks <= 0)
        return fail(FTQ_ERR_INVALID, "bad shape");
    if (num_kv_splits <= 0 || num_kv_splits > 65535)
        return fail(FTQ_ERR_INVALID, "num_kv_splits must be in [1, 65535]");
    if (B == 0) return FTQ_OK;
    if (B > 65535) return fail(FTQ_ERR_INVALID, "B must be at most 65535 per call");
    const bool key_fp8 = key_bits == 8;  // no codebook: centroids_host may be NULL
    const bool key_mse8 = key_bits == FTQ_TQ_KEY_BITS_MSE8;  // centroids_host: 256 entries
    if ((key_fp8 || key_mse8) && value_lloyd_max && value_bits == 4)
        return fail(FTQ_ERR_UNSUPPORTED, "Lloyd-Max value codes need a 4-bit key codebook");
    if (!q || !kv_cache || !block_table || !seq_lens || (!key_fp8 && !centroids_host) || !mid_o || !out)
        return fail(FTQ_ERR_INVALID, "NULL pointer argument");
    if (!aligned(q, 16) || !aligned(out, 4) || !aligned(mid_o, 4))
        return fail(FTQ_ERR_INVALID, "q must be 16-byte aligned, out and mid_o 4-byte aligned");
    if (!aligned(kv_cache, 2) || !even(stride_block) || !even(stride_pos) || !even(stride_head))
        return fail(FTQ_ERR_INVALID, "kv_cache base and strides must be even");
    ftq::TqDecodeParams p{};
    p.q = q;
    p.q_dtype = q_dtype;
    p.B = B;
    p.B_seq = B_seq > 0 ? B_seq : 1;
    p.div_bseq = ftq::make_fastdiv(static_cast<uint32_t>(p.B_seq));
    p.cache_layer_stride = cache_layer_stride;
    p.num_blocks = num_blocks;
    p.Hq = Hq;
    p.Hkv = Hkv;
    p.kv_cache = kv_cache;
    p.stride_block = stride_block;
    p.stride_pos = stride_pos;
    p.stride_head = stride_head;
    p.block_size = block_size;
    p.div_block = ftq::make_fastdiv(static_cast<uint32_t>(block_size));
    p.block_table = block_table;
    p.max_blocks = max_blocks;
    p.seq_lens = seq_lens;
    p.kv_start = kv_start_offset;
    p.norm_correction = norm_correction ? 1 : 0;
    p.value_lloyd_max = (value_lloyd_max && value_bits == 4) ? 1 : 0;  // other widths: ignored, as in the reference
    p.scale = scale;
    p.splits = num_kv_splits;
    const int gh = head_dim == 64 ? 8 : (head_dim == 128 ? 4 : 2);
    p.n_hpass = (Hq / Hkv + gh - 1) / gh;
    if (static_cast<int64_t>(Hkv) * p.n_hpass > 65535) return fail(FTQ_ERR_INVALID, "too many heads");
    p.rsqrt_d = 1.0f / sqrtf(static_cast<float>(head_dim));
    ftq::TqTable256 cent8;
    if (key_mse8) {
        const int rc = pack_table256(centroids_host, 256, false, &cent8);
        if (rc) return rc;
    }
    const ftq::TqTable256* t8 = key_mse8 ? &cent8 : nullptr;
    const int kb = key_mse8 ? 8 : key_bits;
    if (key_fp8 || key_mse8) {
        memset(&p.centroids, 0, sizeof(p.centroids));
    } else {
        const int rc = pack_levels(centroids_host, key_bits, &p.centroids);
        if (rc) return rc;
    }
    p.mid_o = mid_o;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaErrorInvalidValue;
    // 16-bit queries with a GQA group of at most 8 take the tensor-core kernel (head_dim 64 / 128,
    // key and uniform value codes of 2..4 bits); everything else the fp32 kernel
    const int group = Hq / Hkv;
    // (its copy loop reads whole aligned words: a cache that starts on an odd 2-byte boundary -- a
    // view at an offset -- stays on the fp32 kernel, which reads 2-byte pieces)
    const bool mma = q_dtype != FTQ_F32 && group <= 8 && key_bits >= 2 && key_bits <= 4 && value_bits >= 2 &&
                     value_bits != 8 && head_dim != 256 && aligned(kv_cache, 4) &&
                     !p.value_lloyd_max;
    if (mma) {
        // key centroids scaled for the smallest fp16 rounding error of the table (see
        // choose_k_scale).  With norm correction the factor cancels by itself (the centroid
        // vector is re-normalised with the scaled centroids); without, it goes into the
        // softmax scale.
        const float ks = choose_k_scale(centroids_host, key_bits, head_dim);
        for (int i = 0; i < (1 << key_bits); i++) p.centroids.v[i] *= ks;
        if (!p.norm_correction) p.scale = scale / ks;
        const int64_t items = static_cast<int64_t>(B) * Hkv * num_kv_splits;
        if (items >= (1ll << 31)) return fail(FTQ_ERR_INVALID, "too many (sequence, head, split) items");
        const int nh = group <= 4 ? 1 : 2;
        if (head_dim == 64)
            e = ftq::launch_tq_mma_d64(key_bits, value_bits, nh, p, static_cast<int>(items), st);
        else
            e = ftq::launch_tq_mma_d128(key_bits, value_bits, nh, p, static_cast<int>(items), st);
    } else {
        switch (head_dim) {
            case 64: e = ftq::launch_tq_split_d64(kb, value_bits, p, t8, st); break;
            case 128: e = ftq::launch_tq_split_d128(kb, value_bits, p, t8, st); break;
            case 256: e = ftq::launch_tq_split_d256(kb, value_bits, p, t8, st); break;
        }
    }
    if (e != cudaSuccess) return cuda_fail(e, "tq_decode stage 1 launch");
    ftq::TqMergeParams mp{};
    mp.mid_o = mid_o;
    mp.out = out;
    mp.lse = lse;
    mp.n_rows = static_cast<int64_t>(B) * Hq;
    mp.splits = num_kv_splits;
    mp.rotate = rotate_output ? 1 : 0;
    mp.rsqrt_d = p.rsqrt_d;
    mp.prefix_out = prefix_out;
    mp.prefix_dtype = prefix_dtype;
    mp.prefix_lse = prefix_lse;
    switch (head_dim) {
        case 64: e = ftq::launch_tq_merge_d64(out_dtype, mp, st); break;
        case 128: e = ftq::launch_tq_merge_d128(out_dtype, mp, st); break;
        case 256: e = ftq::launch_tq_merge_d256(out_dtype, mp, st); break;
    }
    return e == cudaSuccess ? FTQ_OK : cuda_fail(e, "tq_decode merge launch");
}
