// Memory-bound GQA decode against a static KV cache: split over the sequence, one launch.
//
// The reference has no dedicated decode kernel: a call with few query rows runs the
// prefill kernel's key-lengths variant once per (batch, query head), so a GQA group
// re-reads its K/V head once per query head (aten_attention.cpp:578-604,
// ktt_flash/reader.cpp:111-160). Here the whole group (G query heads x Sq tokens <= 16
// rows) shares one pass over its K/V head, and the passes are cut into equal shares of
// 64-key tiles so that every CTA streams the same number of bytes whatever the
// per-sequence lengths are:
//
//   plan    : every CTA scans ceil(len_b / 64) over the batch into shared memory (the
//             lengths stay on the device; batch <= 512)
//   stream  : CTA c owns the tiles whose unit lies in [c*upc, (c+1)*upc) of the (batch, kv
//             head) pairs laid end to end (a pair's last tile weighs 1 + kPairCost units).
//             K/V rows arrive by 16-byte cp.async into a swizzled ring of stages, one
//             private pipeline per warp (16 keys per tile each), scores and P.V on warp
//             MMA, running max / sum in fp32.
//   finish  : a pair that lies inside one CTA is normalised and written at once. Otherwise
//             each CTA stores its unnormalised partial (O, m, l) in fp32 scratch and takes
//             a ticket on the pair's counter; the CTA that draws the last ticket merges the
//             pair's partials (fixed order: deterministic), writes bf16 and puts the
//             counter back to zero.
//
// Scratch: 1024 int32 ticket counters that must be zero before the first call (the kernel
// leaves them zero), then per slot 16 maxima, 16 sums and 16 x D partial outputs. A pair
// that spans several CTAs is the last pair of the first of them, so that CTA's index names
// its counter: the counter area has one size whatever the batch, and calls of different
// shapes can share one scratch buffer without a partial ever landing on a counter.
//
// Semantics are kohakutt.sdpa(q, k, v, key_lengths=) (attention.py:10-23): keys at or past
// a length contribute nothing, whatever they hold; lengths are clamped to [1, Sk].
#include <mutex>

#include "common.cuh"

namespace ktt {

struct DecodeParams {
    int batch, heads, kv_heads, sq, sk, d;
    float scale_log2;
    const __nv_bfloat16* q;
    const __nv_bfloat16* k;
    const __nv_bfloat16* v;
    __nv_bfloat16* out;
    float* lse;
    int64_t qs[3], ks[3], vs[3], os[3];
    const int32_t* key_lengths;
    int32_t* counters;  // [kMaxCtas] tickets, indexed by the first CTA of a pair; zero between calls
    float* part_m;      // [slots][16]
    float* part_l;      // [slots][16]
    float* part_o;      // [slots][16][d]
    int slots;
    // Append mode (decode_kernel<.., true>): the step's new key / value rows and the rotary
    // rows; k and v above are then written at each sequence's position.
    const __nv_bfloat16* k_new;   // [B, Hk, D]
    const __nv_bfloat16* v_new;
    int64_t kns[2], vns[2];       // (batch, head) strides
    const __nv_bfloat16* rope_cos;
    const __nv_bfloat16* rope_sin;
    int64_t rope_stride;
    int rope_by_position;
    int32_t* lengths_out;
    long long* trace;   // optional (ktt_b200_set_trace): per CTA, nanosecond stamps of its phases
};

namespace {

constexpr int kTile = 64;      // keys per tile (16 per warp)
constexpr int kThreads = 128;
constexpr int kMaxBatch = 512;   // clamped lengths and their prefix sums live in shared memory
constexpr int kMaxPending = 8;   // stored partials per CTA before their tickets are drawn
// Ending a (batch, kv head) pair costs a CTA about as much as streaming five tiles (the four
// warps' states are merged, the result or a partial is written, a ticket may be drawn, the
// next pair's query is fetched): the shares are cut in units in which a pair's last tile
// weighs 1 + kPairCost. Measured on B 64, lengths U[512, 4096], D 128: 36.3, 35.4, 35.0,
// 34.6, 34.5, 34.9 us for a cost of 1 to 6 with every ticket drawn at a CTA's end; 34.95,
// 34.25, 33.8, 34.4 us for 3 to 6 with a finished pair's ticket drawn in mid-stream.
#ifndef KTT_DECODE_PAIR_COST
#define KTT_DECODE_PAIR_COST 5
#endif
constexpr int kPairCost = KTT_DECODE_PAIR_COST;
constexpr int kMaxCtas = 1024;   // ticket counters in the scratch

// Keys batch b attends over. Append mode: the cached count clamped to [0, sk - 1], plus the
// new key.
template <bool kAppend>
__device__ __forceinline__ int clamp_len(const DecodeParams& p, int b) {
    if (kAppend) {
        int l = p.key_lengths[b];
        l = l < 0 ? 0 : l;
        return (l > p.sk - 1 ? p.sk - 1 : l) + 1;
    }
    if (!p.key_lengths) return p.sk;
    int l = p.key_lengths[b];
    l = l < 1 ? 1 : l;
    return l > p.sk ? p.sk : l;
}

// Rotate-half rotary embedding of columns c, c + 1 of a row x (c even): products and sum
// rounded separately in fp32, as the composite op does.
template <int D>
__device__ __forceinline__ uint32_t rope_pair(const __nv_bfloat16* x, const __nv_bfloat16* cs,
                                              const __nv_bfloat16* sn, int c) {
    const bool low = c < D / 2;
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + c));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + (low ? c + D / 2 : c - D / 2)));
    const float2 co = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(cs + c));
    const float2 si = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(sn + c));
    const float r0 = low ? -b.x : b.x, r1 = low ? -b.y : b.y;
    return pack_bf16(__fadd_rn(__fmul_rn(a.x, co.x), __fmul_rn(r0, si.x)),
                     __fadd_rn(__fmul_rn(a.y, co.y), __fmul_rn(r1, si.y)));
}

// prefix[b] = sum_{b' < b} (ceil(len_b' / 64) + kPairCost) for b in [0, batch], by one CTA of
// 128 threads: the units of one kv head's pass over batch entries [0, b).
template <bool kAppend>
__device__ __forceinline__ void scan_lengths(const DecodeParams& p, int* prefix, int* lens, int* warp_sums) {
    constexpr int kPer = kMaxBatch / kThreads;  // consecutive entries per thread
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int tiles[kPer], mine = 0;
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
        const int b = threadIdx.x * kPer + i;
        const int len = b < p.batch ? clamp_len<kAppend>(p, b) : 0;
        if (b < p.batch) lens[b] = len;
        tiles[i] = b < p.batch ? (len + kTile - 1) / kTile + kPairCost : 0;
        mine += tiles[i];
    }
    int x = mine;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, x, off);
        if (lane >= off) x += y;
    }
    if (lane == 31) warp_sums[warp] = x;
    __syncthreads();
    int before = x - mine;
    for (int w = 0; w < warp; ++w) before += warp_sums[w];
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
        const int b = threadIdx.x * kPer + i;
        if (b <= p.batch) prefix[b] = before;
        before += tiles[i];
    }
    if (threadIdx.x == kThreads - 1 && p.batch == kMaxBatch) prefix[kMaxBatch] = before;
    __syncthreads();
}

// Position inside the end-to-end sequence of (batch, kv head) pairs.
struct Cursor {
    int b, hk, tile, ntiles, len;
};

// Largest b with kv_heads * prefix[b] <= unit.
__device__ __forceinline__ int entry_of(const DecodeParams& p, const int* prefix, int unit) {
    int lo = 0, hi = p.batch - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (p.kv_heads * prefix[mid] <= unit) lo = mid; else hi = mid - 1;
    }
    return lo;
}

// Tiles whose unit lies before `unit` (a pair's units: its tiles, then kPairCost units that
// belong to its last tile).
__device__ __forceinline__ int tiles_before(const DecodeParams& p, const int* prefix, int unit) {
    const int b = entry_of(p, prefix, unit);
    const int span = prefix[b + 1] - prefix[b], ntiles = span - kPairCost;
    const int rem = unit - p.kv_heads * prefix[b];
    const int hk = rem / span, pos = rem % span;
    return p.kv_heads * (prefix[b] - kPairCost * b) + hk * ntiles + min(pos, ntiles);
}

// The first tile at or after `unit`.
__device__ __forceinline__ void cursor_seek(const DecodeParams& p, const int* prefix, const int* lens, Cursor& c, int unit) {
    const int b = entry_of(p, prefix, unit);
    const int span = prefix[b + 1] - prefix[b];
    c.b = b;
    c.ntiles = span - kPairCost;
    c.len = lens[b];
    const int rem = unit - p.kv_heads * prefix[b];
    c.hk = rem / span;
    c.tile = rem % span;
    if (c.tile >= c.ntiles) {   // inside a pair's closing units: the next pair's first tile
        c.tile = 0;
        if (++c.hk == p.kv_heads) {
            c.hk = 0;
            if (++c.b < p.batch) {
                c.len = lens[c.b];
                c.ntiles = prefix[c.b + 1] - prefix[c.b] - kPairCost;
            }
        }
    }
}

__device__ __forceinline__ void cursor_next(const DecodeParams& p, const int* prefix, const int* lens, Cursor& c) {
    if (++c.tile < c.ntiles) return;
    c.tile = 0;
    if (++c.hk < p.kv_heads) return;
    c.hk = 0;
    if (++c.b < p.batch) {
        c.len = lens[c.b];
        c.ntiles = prefix[c.b + 1] - prefix[c.b] - kPairCost;
    }
}

// Byte offset of element (row, col) in a [rows][D] bf16 tile whose 16-byte chunks are
// XOR-swizzled by the row, which keeps fragment loads and ldmatrix conflict-free.
template <int D>
__device__ __forceinline__ int swz(int row, int col) {
    return (row * D + ((((col >> 3) ^ (row & 7))) << 3) + (col & 7)) * 2;
}

template <int D, int NS, bool kAppend>
__global__ void __launch_bounds__(kThreads, 2) decode_kernel(const DecodeParams p) {
    constexpr int kStage = 2 * kTile * D * 2;  // K then V, bytes
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* ring = smem;
    float* sm_m = reinterpret_cast<float*>(smem + NS * kStage);  // [4][16]
    float* sm_l = sm_m + 64;                                    // [4][16]
    float* fin_m = sm_l + 64;                                   // [16] merged maxima of a segment
    float* fin_l = fin_m + 16;                                  // [16] merged sums
    int* prefix_s = reinterpret_cast<int*>(fin_l + 16);         // [kMaxBatch + 1]
    int* lens_s = prefix_s + kMaxBatch + 1;                     // [kMaxBatch] clamped lengths
    int* misc = lens_s + kMaxBatch;                       // [8] warp sums, then the pending list

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int group = p.heads / p.kv_heads;
    const int rows = group * p.sq;  // valid rows of the 16-row MMA tile

    // Launched with programmatic stream serialization: the next kernel in the stream may be
    // scheduled while this one drains; nothing here reads global memory before the previous
    // kernel in the stream has completed (a decode loop appends to the cache it reads).
    // Phase stamps (global nanosecond timer) of this CTA when a trace buffer is set: start,
    // after the dependency wait, after the length scan, first tile landed, stream done, end.
    auto stamp = [&](int slot) {
        if (p.trace && threadIdx.x == 0 && blockIdx.x < 1024) {
            long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            p.trace[(64 + blockIdx.x) * 8 + slot] = t;
            if (slot == 0) {
                unsigned smid;
                asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
                p.trace[(64 + blockIdx.x) * 8 + 6] = smid;
            }
        }
    };
    stamp(0);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    stamp(1);

    scan_lengths<kAppend>(p, prefix_s, lens_s, misc);
    stamp(2);
    if (kAppend && blockIdx.x == 0 && p.lengths_out) {
        for (int b = threadIdx.x; b < p.batch; b += kThreads) p.lengths_out[b] = lens_s[b];
    }
    // Equal shares of units; this CTA streams the tiles whose unit lies in its share.
    const int total = p.kv_heads * prefix_s[p.batch];
    const int upc = (total + gridDim.x - 1) / gridDim.x;
    const int first_unit = min(static_cast<int>(blockIdx.x) * upc, total), end_unit = min(first_unit + upc, total);
    const int u0 = 0;
    const int u1 = tiles_before(p, prefix_s, end_unit) - tiles_before(p, prefix_s, first_unit);
    if (u1 <= 0) return;

    Cursor prod, cons;
    cursor_seek(p, prefix_s, lens_s, cons, first_unit);
    prod = cons;

    // One normalised output row chunk (4 columns) of (batch b, kv head hk, tile row r).
    auto write_row = [&](int b, int hk, int r, int c4, float4 sum, float mm, float ll) {
        const float inv = ll > 0.f ? 1.f / ll : 0.f;
        const int gi = r / p.sq, tq = r % p.sq;
        const int h = hk * group + gi;
        __nv_bfloat16* og = p.out + b * p.os[0] + h * p.os[1] + tq * p.os[2] + c4 * 4;
        uint2 packed;
        packed.x = pack_bf16(sum.x * inv, sum.y * inv);
        packed.y = pack_bf16(sum.z * inv, sum.w * inv);
        *reinterpret_cast<uint2*>(og) = packed;
        if (p.lse && c4 == 0) {
            p.lse[(static_cast<int64_t>(b) * p.heads + h) * p.sq + tq] =
                ll > 0.f ? kLn2 * (mm + log2f(ll)) : -INFINITY;
        }
    };

    // Pairs whose partial this CTA has stored and whose ticket it still has to draw.
    int* pend = misc + 8;            // [kMaxPending][5]: pair, first CTA, last CTA, batch, kv head
    int* npend_s = pend + 5 * kMaxPending;
    int* last_s = npend_s + 1;       // [kMaxPending] 1 where this CTA drew the last ticket
    if (threadIdx.x == 0) npend_s[0] = 0;
    __syncthreads();

    // Draws a ticket per pending pair; where this CTA is the last holder it merges the pair's
    // partials (read through L2, fixed order of CTAs: deterministic), writes the rows and
    // puts the counter back to zero for the next call. Called by the whole CTA.
    auto draw_tickets = [&]() {
        __syncthreads();  // every thread's partial stores happen before thread 0's release
        const int n = npend_s[0];
        if (threadIdx.x < n) {
            // One thread per pending pair, so the round trips overlap. An acquire-release RMW
            // at GPU scope publishes this CTA's partials (the barrier above makes the release
            // cumulative over the CTA) and, for the last holder, makes the other holders'
            // partials visible.
            const int* e = pend + 5 * threadIdx.x;
            const int parts = e[2] - e[1] + 1;
            int ticket;
            asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(ticket) : "l"(p.counters + e[1]) : "memory");
            last_s[threadIdx.x] = ticket == parts - 1;
            if (ticket == parts - 1) p.counters[e[1]] = 0;  // all holders have drawn
        }
        __syncthreads();
        // All pairs this CTA finishes, flattened, two positions per thread at a time: the
        // partials of four holders for both positions are requested before any is used, so
        // a thread waits for L2 once per two positions and four holders. (One position at a
        // time, every position's loads waited for the previous position's sums: with two
        // pairs to finish that was four trips to L2 in a row behind the slowest stream.)
        const int per_pair = rows * (D / 4);
        constexpr int kIlp = 2;
        for (int base = 0; base < n * per_pair; base += kIlp * kThreads) {
            bool act[kIlp];
            int r_[kIlp], c4_[kIlp], slot0[kIlp], parts[kIlp], b_[kIlp], hk_[kIlp];
            float mm[kIlp], ll[kIlp];
            float4 sum[kIlp];
            int most = 0;
#pragma unroll
            for (int u = 0; u < kIlp; ++u) {
                const int idx = base + u * kThreads + static_cast<int>(threadIdx.x);
                const int i = idx < n * per_pair ? idx / per_pair : 0;
                act[u] = idx < n * per_pair && last_s[i];
                const int* e = pend + 5 * i;
                const int rem = idx - i * per_pair;
                r_[u] = rem / (D / 4);
                c4_[u] = rem % (D / 4);
                slot0[u] = e[1] + e[0];           // first holder's slot: first CTA + pair
                parts[u] = act[u] ? e[2] - e[1] + 1 : 0;
                b_[u] = e[3];
                hk_[u] = e[4];
                mm[u] = -INFINITY;
                ll[u] = 0.f;
                sum[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                most = max(most, parts[u]);
            }
            // Running merge in CTA order (deterministic), four holders per round.
            for (int c0 = 0; c0 < most; c0 += 4) {
                float ms[kIlp][4], ls[kIlp][4];
                float4 v[kIlp][4];
#pragma unroll
                for (int u = 0; u < kIlp; ++u) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        // Past the last holder (or an idle position): a repeat of a valid slot, not used.
                        const int slot = slot0[u] + max(min(c0 + j, parts[u] - 1), 0);
                        ms[u][j] = __ldcg(&p.part_m[slot * 16 + r_[u]]);
                        ls[u][j] = __ldcg(&p.part_l[slot * 16 + r_[u]]);
                        v[u][j] = __ldcg(reinterpret_cast<const float4*>(p.part_o + (static_cast<int64_t>(slot) * 16 + r_[u]) * D + c4_[u] * 4));
                    }
                }
#pragma unroll
                for (int u = 0; u < kIlp; ++u) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (c0 + j < parts[u]) {
                            const float m_new = fmaxf(mm[u], ms[u][j]);
                            const float base_m = (m_new == -INFINITY) ? 0.f : m_new;
                            const float fa = fast_exp2(mm[u] - base_m), fb = fast_exp2(ms[u][j] - base_m);
                            ll[u] = ll[u] * fa + ls[u][j] * fb;
                            sum[u].x = sum[u].x * fa + v[u][j].x * fb;
                            sum[u].y = sum[u].y * fa + v[u][j].y * fb;
                            sum[u].z = sum[u].z * fa + v[u][j].z * fb;
                            sum[u].w = sum[u].w * fa + v[u][j].w * fb;
                            mm[u] = m_new;
                        }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < kIlp; ++u) {
                if (act[u]) write_row(b_[u], hk_[u], r_[u], c4_[u], sum[u], mm[u], ll[u]);
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) npend_s[0] = 0;
        __syncthreads();
    };

    // One warp copies its own 16 key rows of K and V for a tile into stage `st`.
    auto issue = [&](const Cursor& c, int st) {
        const __nv_bfloat16* kg = p.k + c.b * p.ks[0] + c.hk * p.ks[1];
        const __nv_bfloat16* vg = p.v + c.b * p.vs[0] + c.hk * p.vs[1];
        const uint32_t sk = smem_u32(ring + st * kStage);
        const uint32_t sv = sk + kTile * D * 2;
        constexpr int CH = D / 8;
#pragma unroll
        for (int it = 0; it < 16 * CH / 32; ++it) {
            const int idx = it * 32 + lane;
            const int r = warp * 16 + idx / CH, ch = idx % CH;
            const int j = c.tile * kTile + r;
            const bool ok = j < c.len;
            const int64_t jj = ok ? j : 0;
            cp_async_16(sk + swz<D>(r, ch * 8), kg + jj * p.ks[2] + ch * 8, ok);
            cp_async_16(sv + swz<D>(r, ch * 8), vg + jj * p.vs[2] + ch * 8, ok);
        }
    };

    // Prologue: NS - 1 tiles in flight.
    int up = u0;
#pragma unroll
    for (int s = 0; s < NS - 1; ++s) {
        if (up < u1) {
            issue(prod, s);
            cursor_next(p, prefix_s, lens_s, prod);
            ++up;
        }
        cp_async_commit();
    }

    uint32_t qa[D / 16][4];
    uint32_t k_patch[D / 64], v_patch[D / 64];  // append mode: this lane's share of the new rows
    float o[D / 8][4];
    float m_run[2], l_run[2];
    bool fresh = true;  // start of a pair segment: load Q, reset the running state

    for (int u = u0; u < u1; ++u) {
        const int st = (u - u0) % NS;
        // Refill the stage consumed in the previous iteration.
        if (up < u1) {
            issue(prod, (up - u0) % NS);
            cursor_next(p, prefix_s, lens_s, prod);
            ++up;
        }
        cp_async_commit();

        if (fresh) {
            fresh = false;
            // A-fragments of this pair's query rows: row r = head-in-group * Sq + token.
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int r = g + half * 8;
                const bool ok = r < rows;
                const int gi = ok ? r / p.sq : 0, tq = ok ? r % p.sq : 0;
                const __nv_bfloat16* qg = p.q + cons.b * p.qs[0] +
                    (cons.hk * group + gi) * p.qs[1] + tq * p.qs[2];
                if (kAppend) {
                    // The query gets the rotary row of the new token's position.
                    const int64_t rr = (p.rope_by_position ? cons.len - 1 : cons.b) * p.rope_stride;
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {
                        // Unconditional loads (a row past the group reads row 0 and is
                        // zeroed after): all of them are in flight together.
                        const uint32_t lo = rope_pair<D>(qg, p.rope_cos + rr, p.rope_sin + rr, kk * 16 + t * 2);
                        const uint32_t hi = rope_pair<D>(qg, p.rope_cos + rr, p.rope_sin + rr, kk * 16 + 8 + t * 2);
                        qa[kk][half] = ok ? lo : 0u;
                        qa[kk][half + 2] = ok ? hi : 0u;
                    }
                } else {
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    // Unconditional loads (rows past the group read row 0): nothing orders
                    // them, so they are all in flight together.
                    const uint32_t lo = *reinterpret_cast<const uint32_t*>(qg + kk * 16 + t * 2);
                    const uint32_t hi = *reinterpret_cast<const uint32_t*>(qg + kk * 16 + 8 + t * 2);
                    qa[kk][half] = ok ? lo : 0u;
                    qa[kk][half + 2] = ok ? hi : 0u;
                }
                }
            }
            if (kAppend) {
                // The pair's new key (rotated) and value, fetched with the query so that the
                // warp that later places them does not wait for memory then.
                const __nv_bfloat16* kn = p.k_new + cons.b * p.kns[0] + cons.hk * p.kns[1];
                const __nv_bfloat16* vn = p.v_new + cons.b * p.vns[0] + cons.hk * p.vns[1];
                const int64_t rr = (p.rope_by_position ? cons.len - 1 : cons.b) * p.rope_stride;
#pragma unroll
                for (int i = 0; i < D / 64; ++i) {
                    k_patch[i] = rope_pair<D>(kn, p.rope_cos + rr, p.rope_sin + rr, lane * 2 + i * 64);
                    v_patch[i] = *reinterpret_cast<const uint32_t*>(vn + lane * 2 + i * 64);
                }
            }
#pragma unroll
            for (int n = 0; n < D / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
            m_run[0] = m_run[1] = -INFINITY;
            l_run[0] = l_run[1] = 0.f;
        }
        // (The query loads above are in flight while this waits for the tile.)
        cp_async_wait<NS - 1>();
        __syncwarp();
        if (u == u0) stamp(3);

        if (kAppend) {
            // The warp whose 16 rows hold the new token's slot puts the rotated key and the
            // value there, in the tile it is about to use and in the cache. Whatever the
            // copy brought for that row is replaced; no other CTA or warp touches it.
            const int pos = cons.len - 1;
            if (pos / kTile == cons.tile && (pos % kTile) / 16 == warp) {
                const int r = pos % kTile;
                unsigned char* sK = ring + st * kStage;
                unsigned char* sV = sK + kTile * D * 2;
                __nv_bfloat16* kc = const_cast<__nv_bfloat16*>(p.k) + cons.b * p.ks[0] + cons.hk * p.ks[1] + static_cast<int64_t>(pos) * p.ks[2];
                __nv_bfloat16* vc = const_cast<__nv_bfloat16*>(p.v) + cons.b * p.vs[0] + cons.hk * p.vs[1] + static_cast<int64_t>(pos) * p.vs[2];
#pragma unroll
                for (int i = 0; i < D / 64; ++i) {
                    const int c = lane * 2 + i * 64;
                    *reinterpret_cast<uint32_t*>(sK + swz<D>(r, c)) = k_patch[i];
                    *reinterpret_cast<uint32_t*>(sV + swz<D>(r, c)) = v_patch[i];
                    *reinterpret_cast<uint32_t*>(kc + c) = k_patch[i];
                    *reinterpret_cast<uint32_t*>(vc + c) = v_patch[i];
                }
                __syncwarp();
            }
        }

        const int j0 = cons.tile * kTile + warp * 16;
        if (j0 < cons.len) {
            const unsigned char* sK = ring + st * kStage;
            const unsigned char* sV = sK + kTile * D * 2;
            float s[2][4];
#pragma unroll
            for (int n = 0; n < 2; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
                for (int n = 0; n < 2; ++n) {
                    const int r = warp * 16 + n * 8 + g;
                    const uint32_t b0 = *reinterpret_cast<const uint32_t*>(sK + swz<D>(r, kk * 16 + t * 2));
                    const uint32_t b1 = *reinterpret_cast<const uint32_t*>(sK + swz<D>(r, kk * 16 + 8 + t * 2));
                    mma_bf16(s[n], qa[kk], b0, b1);
                }
            }
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int n = 0; n < 2; ++n) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = j0 + n * 8 + t * 2 + (e & 1);
                    const float x = j < cons.len ? s[n][e] * p.scale_log2 : -INFINITY;
                    s[n][e] = x;
                    mx[e >> 1] = fmaxf(mx[e >> 1], x);
                }
            }
            float alpha[2], m_use[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m_run[r], mx[r]);
                m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;
                alpha[r] = fast_exp2(m_run[r] - m_use[r]);
                m_run[r] = m_new;
                l_run[r] *= alpha[r];
            }
#pragma unroll
            for (int n = 0; n < D / 8; ++n) {
                o[n][0] *= alpha[0];
                o[n][1] *= alpha[0];
                o[n][2] *= alpha[1];
                o[n][3] *= alpha[1];
            }
#pragma unroll
            for (int n = 0; n < 2; ++n) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float pv = fast_exp2(s[n][e] - m_use[e >> 1]);
                    s[n][e] = pv;
                    l_run[e >> 1] += pv;
                }
            }
            uint32_t a[4];
            a[0] = pack_bf16(s[0][0], s[0][1]);
            a[1] = pack_bf16(s[0][2], s[0][3]);
            a[2] = pack_bf16(s[1][0], s[1][1]);
            a[3] = pack_bf16(s[1][2], s[1][3]);
            const uint32_t sv_base = smem_u32(sV);
#pragma unroll
            for (int n2 = 0; n2 < D / 16; ++n2) {
                uint32_t r[4];
                ldmatrix_x4_trans(r, sv_base + swz<D>(warp * 16 + (lane & 15), n2 * 16 + (lane >> 4) * 8));
                mma_bf16(o[2 * n2], a, r[0], r[1]);
                mma_bf16(o[2 * n2 + 1], a, r[2], r[3]);
            }
        }
        __syncwarp();  // all lanes are done with stage `st` before it is refilled

        const bool last_of_pair = cons.tile + 1 == cons.ntiles;
        if (last_of_pair || u + 1 == u1) {
            const long long fin_t0 = p.trace ? clock64() : 0;
            // Merge the four warps' states in a fixed order (deterministic).
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
                l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
            }
            if (t == 0) {
                sm_m[warp * 16 + g] = m_run[0];
                sm_m[warp * 16 + g + 8] = m_run[1];
                sm_l[warp * 16 + g] = l_run[0];
                sm_l[warp * 16 + g + 8] = l_run[1];
            }
            __syncthreads();
            float f[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int row = g + r * 8;
                float mm = -INFINITY;
#pragma unroll
                for (int w = 0; w < 4; ++w) mm = fmaxf(mm, sm_m[w * 16 + row]);
                const float base = (mm == -INFINITY) ? 0.f : mm;
                float ll = 0.f;
#pragma unroll
                for (int w = 0; w < 4; ++w) ll += sm_l[w * 16 + row] * fast_exp2(sm_m[w * 16 + row] - base);
                if (warp == 0 && t == 0) {
                    fin_m[row] = mm;
                    fin_l[row] = ll;
                }
                f[r] = fast_exp2(m_run[r] - base);
            }
            // Every warp leaves its rescaled 16 x D fp32 block in its own quarter of the stage
            // it has just consumed (rows 0-7 where its 16 key rows were, rows 8-15 where its
            // value rows were: no other warp reads or refills those bytes), all four at once;
            // after one barrier the CTA adds the four blocks, warp 0's first (a fixed order:
            // deterministic), and writes each sum straight to where it goes.
            constexpr int kQuarter = 16 * D * 2;   // bytes of a warp's rows in a K or V tile
            unsigned char* slab = ring + st * kStage + warp * kQuarter;
#pragma unroll
            for (int n = 0; n < D / 8; ++n) {
                const int col = (n * 8 + t * 2) ^ (g << 3);   // rows spread over the banks
                *reinterpret_cast<float2*>(slab + (g * D + col) * 4) = make_float2(o[n][0] * f[0], o[n][1] * f[0]);
                *reinterpret_cast<float2*>(slab + kTile * D * 2 + (g * D + col) * 4) = make_float2(o[n][2] * f[1], o[n][3] * f[1]);
            }
            __syncthreads();
            auto merged = [&](int r, int c4) {
                const unsigned char* base = ring + st * kStage + (r >= 8 ? kTile * D * 2 : 0) + (((r & 7) * D + ((c4 * 4) ^ ((r & 7) << 3))) * 4);
                float4 sum = *reinterpret_cast<const float4*>(base);
#pragma unroll
                for (int w = 1; w < 4; ++w) {
                    const float4 x = *reinterpret_cast<const float4*>(base + w * kQuarter);
                    sum.x += x.x;
                    sum.y += x.y;
                    sum.z += x.z;
                    sum.w += x.w;
                }
                return sum;
            };

            // Which CTAs hold a piece of this pair?
            const int pair = cons.b * p.kv_heads + cons.hk;
            const int t0 = p.kv_heads * prefix_s[cons.b] + cons.hk * (cons.ntiles + kPairCost);   // the pair's first unit
            const int c_first = t0 / upc, c_last = (t0 + cons.ntiles - 1) / upc;
            if (c_first == c_last) {
                // The whole pair lies in this CTA: normalise and write it now.
                for (int idx = threadIdx.x; idx < rows * (D / 4); idx += kThreads) {
                    const int r = idx / (D / 4), c4 = idx % (D / 4);
                    write_row(cons.b, cons.hk, r, c4, merged(r, c4), fin_m[r], fin_l[r]);
                }
            } else {
                // Store the partial and note the ticket to draw.
                const int slot = blockIdx.x + pair;
                float4* dst = reinterpret_cast<float4*>(p.part_o + static_cast<int64_t>(slot) * 16 * D);
                for (int idx = threadIdx.x; idx < rows * D / 4; idx += kThreads) dst[idx] = merged(idx / (D / 4), idx % (D / 4));
                if (threadIdx.x < 16) {
                    p.part_m[slot * 16 + threadIdx.x] = fin_m[threadIdx.x];
                    p.part_l[slot * 16 + threadIdx.x] = fin_l[threadIdx.x];
                }
                if (threadIdx.x == 0) {
                    int* e = pend + 5 * npend_s[0];
                    e[0] = pair; e[1] = c_first; e[2] = c_last; e[3] = cons.b; e[4] = cons.hk;
                    npend_s[0] += 1;
                }
                __syncthreads();
                // A pair that ends in the middle of this CTA's share draws its ticket now: the
                // other holder of that pair is then almost always the last one, so a CTA ends
                // with one pair to merge, not with whichever pairs it happened to finish last
                // (the three-stage ring rides out the fence; measured 34.6 -> 34.25 us, and
                // 33.8 us with the pair cost re-swept).
                if (npend_s[0] == kMaxPending || u + 1 < u1) draw_tickets();
            }
            __syncthreads();
            fresh = true;
            if (p.trace && threadIdx.x == 0 && blockIdx.x < 1024) p.trace[(64 + blockIdx.x) * 8 + 7] += clock64() - fin_t0;
        }
        cursor_next(p, prefix_s, lens_s, cons);
    }
    cp_async_wait<0>();
    __syncthreads();
    stamp(4);
    if (npend_s[0] > 0) draw_tickets();
    stamp(5);
}

int stream_ctas_for_device() {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) {
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    }
    return 2 * sms;
}

template <int D, int NS, bool kAppend>
int launch(const DecodeParams& p, int ctas, cudaStream_t stream) {
    constexpr int smem = NS * 2 * kTile * D * 2 + (2 * 64 + 32) * 4 + (2 * kMaxBatch + 1 + 8 + 6 * kMaxPending + 1) * 4;
    if (int rc = ensure_smem(decode_kernel<D, NS, kAppend>, smem, "cudaFuncSetAttribute(decode)")) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(ctas));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return check_cuda(cudaLaunchKernelEx(&cfg, decode_kernel<D, NS, kAppend>, p), "decode launch");
}

// Scratch layout: 1024 ticket counters (int32), then m, l, O partials.
struct ScratchLayout {
    int64_t counter_bytes, m_bytes, l_bytes, o_bytes, total;
    int slots;
};

ScratchLayout scratch_layout(int batch, int kv_heads, int d, int ctas) {
    ScratchLayout s;
    s.slots = ctas + batch * kv_heads;
    auto up = [](int64_t x) { return (x + 255) / 256 * 256; };
    s.counter_bytes = kMaxCtas * 4;
    s.m_bytes = up(static_cast<int64_t>(s.slots) * 16 * 4);
    s.l_bytes = s.m_bytes;
    s.o_bytes = up(static_cast<int64_t>(s.slots) * 16 * d * 4);
    s.total = s.counter_bytes + s.m_bytes + s.l_bytes + s.o_bytes;
    return s;
}

int decode_ctas(const ktt_b200_decode_args* a) {
    // `splits` bounds the CTAs per (batch, kv head) pair; 0 lets the device size decide.
    int ctas = stream_ctas_for_device();
    if (a->splits > 0) {
        const int64_t want = static_cast<int64_t>(a->splits) * a->batch * a->kv_heads;
        if (want < ctas) ctas = static_cast<int>(want);
    }
    if (ctas > kMaxCtas) ctas = kMaxCtas;
    return ctas < 1 ? 1 : ctas;
}

const char* decode_refusal(const ktt_b200_decode_args* a) {
    if (!a) return "null arguments";
    if (a->batch < 1 || a->heads < 1 || a->kv_heads < 1 || a->sq < 1 || a->sk < 1) return "sizes must be positive";
    if (a->batch > kMaxBatch) return "decode takes at most 512 sequences per call";
    if (a->heads % a->kv_heads) return "K / V heads must divide Q heads";
    if (a->d != a->dv || (a->d != 64 && a->d != 128)) return "decode takes head dim 64 or 128 (D == Dv)";
    if ((a->heads / a->kv_heads) * a->sq > 16) return "decode takes at most 16 query rows per K / V head";
    for (int i = 0; i < 3; ++i) {
        if (a->k_strides[i] % 8 || a->v_strides[i] % 8) return "K / V strides must be multiples of 8 elements";
        if (a->q_strides[i] % 2 || a->out_strides[i] % 4) return "q strides must be even and out strides multiples of 4";
    }
    return nullptr;
}

// Checks, parameter block and launch shared by both entry points; `base` is the scratch.
int run_decode(const ktt_b200_decode_args* a, unsigned char* base, const ScratchLayout& lay, int ctas,
               void* stream, const char* what, const ktt_b200_decode_append_args* app = nullptr) {
    if ((reinterpret_cast<uintptr_t>(a->k) | reinterpret_cast<uintptr_t>(a->v) | reinterpret_cast<uintptr_t>(base)) & 15) {
        return fail(KTT_B200_ERR_UNSUPPORTED, "%s: k, v and scratch must be 16-byte aligned", what);
    }
    if ((reinterpret_cast<uintptr_t>(a->q) & 3) || (reinterpret_cast<uintptr_t>(a->out) & 7)) {
        return fail(KTT_B200_ERR_UNSUPPORTED, "%s: q must be 4-byte and out 8-byte aligned", what);
    }
    DecodeParams p;
    p.batch = a->batch; p.heads = a->heads; p.kv_heads = a->kv_heads;
    p.sq = a->sq; p.sk = a->sk; p.d = a->d;
    p.scale_log2 = a->scale * kLog2e;
    p.q = static_cast<const __nv_bfloat16*>(a->q);
    p.k = static_cast<const __nv_bfloat16*>(a->k);
    p.v = static_cast<const __nv_bfloat16*>(a->v);
    p.out = static_cast<__nv_bfloat16*>(a->out);
    p.lse = a->lse;
    for (int i = 0; i < 3; ++i) {
        p.qs[i] = a->q_strides[i]; p.ks[i] = a->k_strides[i];
        p.vs[i] = a->v_strides[i]; p.os[i] = a->out_strides[i];
    }
    p.key_lengths = a->key_lengths;
    p.counters = reinterpret_cast<int32_t*>(base);
    p.part_m = reinterpret_cast<float*>(base + lay.counter_bytes);
    p.part_l = reinterpret_cast<float*>(base + lay.counter_bytes + lay.m_bytes);
    p.part_o = reinterpret_cast<float*>(base + lay.counter_bytes + lay.m_bytes + lay.l_bytes);
    p.slots = lay.slots;
    p.k_new = p.v_new = p.rope_cos = p.rope_sin = nullptr;
    p.lengths_out = nullptr;
    p.trace = get_trace_buffer();
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    note_call(3);
    if (app) {
        p.k_new = static_cast<const __nv_bfloat16*>(app->k_new);
        p.v_new = static_cast<const __nv_bfloat16*>(app->v_new);
        for (int i = 0; i < 2; ++i) {
            p.kns[i] = app->k_new_strides[i];
            p.vns[i] = app->v_new_strides[i];
        }
        p.rope_cos = static_cast<const __nv_bfloat16*>(app->cos);
        p.rope_sin = static_cast<const __nv_bfloat16*>(app->sin);
        p.rope_stride = app->rope_row_stride;
        p.rope_by_position = app->rope_by_position;
        p.lengths_out = app->lengths_out;
        if (a->d == 64) return launch<64, 6, true>(p, ctas, st);
        return launch<128, 3, true>(p, ctas, st);
    }
    if (a->d == 64) return launch<64, 6, false>(p, ctas, st);
    return launch<128, 3, false>(p, ctas, st);
}

}  // namespace

}  // namespace ktt

using namespace ktt;

extern "C" int64_t ktt_b200_decode_scratch_bytes(const ktt_b200_decode_args* a) {
    if (const char* why = decode_refusal(a)) {
        fail(KTT_B200_ERR_UNSUPPORTED, "decode: %s", why);
        return 0;
    }
    return scratch_layout(a->batch, a->kv_heads, a->d, decode_ctas(a)).total;
}

extern "C" int ktt_b200_decode(const ktt_b200_decode_args* a, void* stream) {
    if (const char* why = decode_refusal(a)) return fail(KTT_B200_ERR_UNSUPPORTED, "decode: %s", why);
    if (!a->q || !a->k || !a->v || !a->out || !a->scratch) {
        return fail(KTT_B200_ERR_BAD_ARGUMENT, "decode: null tensor or scratch pointer");
    }
    const int ctas = decode_ctas(a);
    const ScratchLayout lay = scratch_layout(a->batch, a->kv_heads, a->d, ctas);
    if (a->scratch_bytes < lay.total) {
        return fail(KTT_B200_ERR_BAD_ARGUMENT, "decode: scratch holds %lld bytes, %lld needed",
                    static_cast<long long>(a->scratch_bytes), static_cast<long long>(lay.total));
    }
    return run_decode(a, static_cast<unsigned char*>(a->scratch), lay, ctas, stream, "decode");
}

// One decode step with rotary, cache append and attention in the same launch.
extern "C" int ktt_b200_decode_append(const ktt_b200_decode_append_args* app, void* stream) {
    if (!app) return fail(KTT_B200_ERR_BAD_ARGUMENT, "decode_append: null arguments");
    const ktt_b200_decode_args* a = &app->base;
    if (const char* why = decode_refusal(a)) return fail(KTT_B200_ERR_UNSUPPORTED, "decode_append: %s", why);
    if (a->sq != 1) return fail(KTT_B200_ERR_UNSUPPORTED, "decode_append: one query token per sequence");
    if (!a->q || !a->k || !a->v || !a->out || !a->scratch || !a->key_lengths || !app->k_new || !app->v_new ||
        !app->cos || !app->sin) {
        return fail(KTT_B200_ERR_BAD_ARGUMENT, "decode_append: null tensor, lengths, rotary or scratch pointer");
    }
    if (app->lengths_out == a->key_lengths) {
        return fail(KTT_B200_ERR_BAD_ARGUMENT, "decode_append: lengths_out must not be the lengths themselves");
    }
    const uintptr_t small = reinterpret_cast<uintptr_t>(app->k_new) | reinterpret_cast<uintptr_t>(app->v_new) |
                            reinterpret_cast<uintptr_t>(app->cos) | reinterpret_cast<uintptr_t>(app->sin);
    if ((small & 3) || (app->rope_row_stride & 1) || ((app->k_new_strides[0] | app->k_new_strides[1] |
        app->v_new_strides[0] | app->v_new_strides[1]) & 1)) {
        return fail(KTT_B200_ERR_UNSUPPORTED, "decode_append: new rows and rotary rows must be 4-byte aligned with even strides");
    }
    const int ctas = decode_ctas(a);
    const ScratchLayout lay = scratch_layout(a->batch, a->kv_heads, a->d, ctas);
    if (a->scratch_bytes < lay.total) {
        return fail(KTT_B200_ERR_BAD_ARGUMENT, "decode_append: scratch holds %lld bytes, %lld needed",
                    static_cast<long long>(a->scratch_bytes), static_cast<long long>(lay.total));
    }
    return run_decode(a, static_cast<unsigned char*>(a->scratch), lay, ctas, stream, "decode_append", app);
}

// ---- decode without any allocation ---------------------------------------------------------
//
// Some hosts of this library may not allocate device memory once they are running: an
// inference server that carves up the whole GPU at start-up and hands its plugins nothing
// but input and output buffers, or a decode loop with a latency budget in which a
// cudaMalloc (which can stall the whole device) is not acceptable. For them the split-K
// partials live in a fixed array that is part of the loaded module instead of in
// caller-provided scratch.

namespace ktt {
namespace {

// Room for the partials of 207 (batch, kv head) pairs at head dim 128 on a 148-SM part,
// or 696 pairs at head dim 64. Each GPU that loads the library holds these 4 MiB until
// the process exits.
constexpr int64_t kStaticScratchBytes = 4ll << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of g_static_scratch on the current device. In host code the array's name
// is only a handle for the runtime, not an address a kernel can use, so the address is
// asked for once per device (with that device current) and kept.
int static_scratch_address(unsigned char** out) {
    static std::mutex mutex;
    static unsigned char* address[64] = {};
    int dev = 0;
    if (int rc = check_cuda(cudaGetDevice(&dev), "decode_static: cudaGetDevice")) return rc;
    if (dev < 0 || dev >= 64) return fail(KTT_B200_ERR_UNSUPPORTED, "decode_static: device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(mutex);
    if (!address[dev]) {
        void* ptr = nullptr;
        if (int rc = check_cuda(cudaGetSymbolAddress(&ptr, g_static_scratch), "decode_static: cudaGetSymbolAddress")) {
            return rc;
        }
        address[dev] = static_cast<unsigned char*>(ptr);
    }
    *out = address[dev];
    return 0;
}

}  // namespace
}  // namespace ktt

// Same computation as ktt_b200_decode with the split-K partials in the library's own fixed
// device array: no cudaMalloc, cudaFree or other allocating call is made, here or below.
// args->scratch and args->scratch_bytes are ignored.
//
// Limits and rules:
//  - The partials of the call must fit 4 MiB (see kStaticScratchBytes); a larger problem is
//    refused with KTT_B200_ERR_UNSUPPORTED and a message that names both sizes. Use
//    ktt_b200_decode with caller scratch for those.
//  - The first call on each device looks up the array's device address and raises the
//    kernel's shared-memory limit. Make that first call outside of any stream capture.
//  - All calls on a device share the one array. Nothing in it has to be cleared between
//    calls (the array starts zeroed with the module, the ticket counters are put back to
//    zero by the kernel, every other word is written before it is read), but two calls whose kernels
//    overlap on the GPU, for example on different streams, overwrite each other's
//    partials. Keep calls to this entry point on one stream, or order them with events.
extern "C" int ktt_b200_decode_static(const ktt_b200_decode_args* a, void* stream) {
    if (const char* why = decode_refusal(a)) return fail(KTT_B200_ERR_UNSUPPORTED, "decode_static: %s", why);
    if (!a->q || !a->k || !a->v || !a->out) {
        return fail(KTT_B200_ERR_BAD_ARGUMENT, "decode_static: null tensor pointer");
    }
    const int ctas = decode_ctas(a);
    const ScratchLayout lay = scratch_layout(a->batch, a->kv_heads, a->d, ctas);
    if (lay.total > kStaticScratchBytes) {
        return fail(KTT_B200_ERR_UNSUPPORTED,
                    "decode_static: this call needs %lld bytes of split-K partials, the built-in array holds %lld; "
                    "use ktt_b200_decode with caller-provided scratch",
                    static_cast<long long>(lay.total), static_cast<long long>(kStaticScratchBytes));
    }
    unsigned char* base = nullptr;
    if (int rc = static_scratch_address(&base)) return rc;
    return run_decode(a, base, lay, ctas, stream, "decode_static");
}
