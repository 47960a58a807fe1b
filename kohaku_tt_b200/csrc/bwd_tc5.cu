// Backward on the Blackwell tensor path: dK/dV CTAs and dQ CTAs (two bodies, one launch: see
// bwd_tc5_kernel), both TMA loads + tcgen05.mma with accumulators in tensor memory.
//
// Same split and same arithmetic as the reference's backward (ktt_flash/program.cpp:
// 1587-2006; bw_dq_compute.cpp, bw_dkv_compute.cpp): every gradient has one owner, nothing
// is accumulated with atomics, so results are deterministic and a packed sequence's
// gradients do not depend on its neighbours. With delta_i = sum_d dO_id O_id from the
// preprocess kernel and lse from the forward:
//
//   P = 2^(S scale log2e - lse log2e),  dP = dO V^T,  dS = P o (dP - delta)
//
//   dK/dV kernel  one CTA = 128 keys of one K/V head; it streams the query blocks of every
//                 query head of the group. Everything is computed transposed so that the CTA's
//                 keys are the TMEM lanes:  S^T = K Q^T,  dP^T = V dO^T  (both operands from
//                 shared memory), then P^T and dS^T are written back over S^T and dP^T as
//                 packed bf16 and feed  dV += P^T dO,  dK += dS^T Q  as the A operand from
//                 tensor memory (dO and Q are the MN-major B operands). dV and dK stay in
//                 TMEM for the whole loop: there is no running maximum to rescale by.
//   dQ kernel     one CTA = 128 query rows of one head; it streams key blocks:
//                 S = Q K^T,  dP = dO V^T,  dS over dP in place,  dQ += dS K  (K is read as
//                 the K-major B operand of the first MMA and as the MN-major B operand of
//                 the last one, from the same tile).
//
// Ten warps per CTA: warps 0-7 are two groups of 128 threads (one thread per TMEM lane, each
// group owning 64 of the block's 128 score columns), warp 8 issues MMAs, warp 9 issues TMA.
// Every wait is a bounded mbarrier wait as in the forward kernel, the meetings of the score
// warps included. Optional per call: key lengths, a mask of one row per (batch, head).
//
// Overlap: the scores have two buffers in tensor memory wherever 128 columns are left (the dQ
// kernel at both head dims, the dK/dV kernel at D 64), so the score MMA of item i + 1 runs
// while the threads still work on item i; dP has one buffer (dS is written over it and read
// by the last MMA of the item), so dP of item i + 1 is issued behind that MMA and arrives
// while the threads exponentiate the scores of item i + 1. A thread therefore works in two
// phases per item: scores -> P (kept in registers, in the dK/dV kernel also stored as the
// operand of dV), then dP -> dS.
#include "tc5.cuh"

namespace ktt {
using namespace tc5;
namespace {

constexpr int kThreads = 320;
// Exponentials per 8 pairs that take the FMA-pipe polynomial instead of MUFU, spread evenly.
#ifndef KTT_BWD_POLY_PAIRS
#define KTT_BWD_POLY_PAIRS 2
#endif
__host__ __device__ constexpr bool poly_pair(int pair) {
    return ((pair % 8) * KTT_BWD_POLY_PAIRS) % 8 < KTT_BWD_POLY_PAIRS && KTT_BWD_POLY_PAIRS > 0;
}
constexpr int kTmemCols = 512;

struct BwdParams {
    AttnParams a;
    int* status;
    int dim_of[4][3];  // q, k, v, dout: tensor-map coordinate slot of row, head, batch
    long long* trace;  // optional (ktt_b200_set_trace): per-CTA start / end / SM
    Divisor by_dkv_x, by_dkv_y, by_dq_x, by_dq_y, by_gsplit, by_group;   // group: query heads per kv head
};


// Shared-memory plan: a resident pair of tiles (A0, A1), a ring of streamed pairs (B0, B1),
// two double-buffered vectors of 128 floats, barriers.
template <int D>
struct BwdPlan {
    static constexpr int kSub = D / 64;
    static constexpr int kTile = 128 * 128;              // one [128][64] bf16 sub-tile
    static constexpr int kStages = D == 64 ? 4 : 2;
    static constexpr int kA0 = 0;
    static constexpr int kA1 = kA0 + kSub * kTile;
    static constexpr int kB0 = kA1 + kSub * kTile;
    static constexpr int kB1 = kB0 + kStages * kSub * kTile;
    static constexpr int kVec = kB1 + kStages * kSub * kTile;  // float [3 buffers][2 vectors][128] (dK/dV), [2][128] mask terms (dQ)
    static constexpr int kBars = kVec + 2 * 3 * 128 * 4;
    static constexpr int kBytes = kBars + 256;
    static constexpr int bAFull = 0;
    static constexpr int bBFull = 1;                  // + stage
    static constexpr int bBEmpty = bBFull + kStages;  // + stage
    static constexpr int bSReady = bBEmpty + kStages; // + score buffer
    static constexpr int bDPReady = bSReady + 2;
    static constexpr int bPFull = bDPReady + 1;       // + half
    static constexpr int bDone = bPFull + 2;
    static constexpr int bMeet = bDone + 1;           // the eight score warps meet (bounded, unlike bar.sync)
    static constexpr int bCount = bMeet + 1;
    static_assert(bCount * 8 + 16 <= 256, "barrier area");
};

template <int D>
__device__ __forceinline__ void init_barriers(uint32_t bars, volatile int* abort_flag) {
    using P = BwdPlan<D>;
    mbar_init(bars + 8 * P::bAFull, 1);
    for (int s = 0; s < P::kStages; ++s) {
        mbar_init(bars + 8 * (P::bBFull + s), 1);
        mbar_init(bars + 8 * (P::bBEmpty + s), 1);
    }
    mbar_init(bars + 8 * (P::bSReady + 0), 1);
    mbar_init(bars + 8 * (P::bSReady + 1), 1);
    mbar_init(bars + 8 * P::bDPReady, 1);
    mbar_init(bars + 8 * (P::bPFull + 0), 4);   // one arrival per warp of the group
    mbar_init(bars + 8 * (P::bPFull + 1), 4);
    mbar_init(bars + 8 * P::bDone, 1);
    mbar_init(bars + 8 * P::bMeet, 8);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
}

// Phase stamp of a CTA's first thread (slots 4..7 of its trace row), while a buffer is set.
__device__ __forceinline__ void mark(const BwdParams& tp, int slot) {
    if (tp.trace && threadIdx.x == 0 && blockIdx.x < 1024) {
        long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        tp.trace[(64 + blockIdx.x) * 8 + slot] = t;
    }
}

// ---- dK / dV ----------------------------------------------------------------------------

// Body of one dK/dV CTA; (bx, by, bz) = (kv head * gsplit + part, key block, batch).
template <int D, bool kMask>
__device__ __forceinline__ void dkv_body(
    const CUtensorMap* pmap_q, const CUtensorMap* pmap_k, const CUtensorMap* pmap_v, const CUtensorMap* pmap_do,
    const BwdParams& tp, int bx, int by, int bz, int gridDim_y) {
    const CUtensorMap& map_q = *pmap_q;
    const CUtensorMap& map_k = *pmap_k;
    const CUtensorMap& map_v = *pmap_v;
    const CUtensorMap& map_do = *pmap_do;
    using P = BwdPlan<D>;
    extern __shared__ __align__(1024) unsigned char smem[];
    const uint32_t sbase = smem_u32(smem);
    if (sbase & 1023u) {
        if (threadIdx.x == 0) atomicCAS_system(tp.status, 0, 901);
        return;
    }
    const uint32_t bars = sbase + P::kBars;
    auto bar = [&](int i) { return bars + 8u * i; };
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + P::kBars + P::bCount * 8);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + P::kBars + P::bCount * 8 + 8);
    float* vec = reinterpret_cast<float*>(smem + P::kVec);  // [item mod 3][0: lse2, 1: delta][128]

    const AttnParams& p = tp.a;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // blockIdx.x = kv head * gsplit + part: this CTA handles query heads [g0, g0 + group) of
    // the kv head's GQA group.
    const int hk = div_by(bx, tp.by_gsplit), part = bx - hk * p.gsplit, kb = by, b = bz;
    const SeqInfo si = seq_info(p, b);
    const int k0 = kb * kBM;
    if (k0 >= si.lk) return;
    const int full_group = static_cast<int>(tp.by_group.d);
    const int g0 = div_by(part * full_group, tp.by_gsplit);
    const int group = div_by((part + 1) * full_group, tp.by_gsplit) - g0;
    const int nq = (si.lq + kBN - 1) / kBN;
    int qstart = 0;
    if (p.causal) {
        const int first = k0 - si.shift;  // first query row that can see key k0
        qstart = first > 0 ? first / kBN : 0;
    }
    const bool any_key = k0 < si.klen;
    const int per_head = (any_key && nq > qstart) ? nq - qstart : 0;
    const int nitems = per_head * group;

    auto coords = [&](int operand, int row, int head, int batch, int (&c)[4]) {
        c[tp.dim_of[operand][0]] = row;
        c[tp.dim_of[operand][1]] = head;
        c[tp.dim_of[operand][2]] = batch;
    };
    const int batch_c = p.cu_q ? 0 : b;
    // Q and dO tiles of item `it` into their ring stage (producer warp, converged; called for
    // it = 0, 1, 2, ... in turn, so head and query block are counted, not divided out).
    int ld_head = 0, ld_qb = 0;
    auto load_item = [&](int it) {
        int c[4], c2[4];
        c[0] = c2[0] = 0;
        const int st = it % P::kStages;
        const int h = hk * full_group + g0 + ld_head;
        const int q0 = (qstart + ld_qb) * kBN;
        if (++ld_qb == per_head) {
            ld_qb = 0;
            ++ld_head;
        }
        coords(0, si.q_off + q0, h, batch_c, c);
        coords(3, si.q_off + q0, h, batch_c, c2);
        mbar_expect_tx(bar(P::bBFull + st), 2 * P::kSub * P::kTile);
        for (int s = 0; s < P::kSub; ++s) {
            tma_load_4d(sbase + P::kB0 + (st * P::kSub + s) * P::kTile, &map_q, bar(P::bBFull + st), s * 64, c[1], c[2], c[3]);
            tma_load_4d(sbase + P::kB1 + (st * P::kSub + s) * P::kTile, &map_do, bar(P::bBFull + st), s * 64, c2[1], c2[2], c2[3]);
        }
    };

    // Set-up. The producer warp initialises the barriers itself and sends the CTA's first
    // loads (K, V and the first ring stages; none of them is written by the delta kernel this
    // launch may overlap) while warp 8 allocates tensor memory and the rest wait.
    int issued = 0;
    if (warp == 9) {
        if (lane == 0) init_barriers<D>(bars, abort_flag);
        __syncwarp();
        if (nitems > 0) {
            int c[4], c2[4];
            c[0] = c2[0] = 0;
            coords(1, si.k_off + k0, hk, batch_c, c);
            coords(2, si.k_off + k0, hk, batch_c, c2);
            mbar_expect_tx(bar(P::bAFull), 2 * P::kSub * P::kTile);
            for (int s = 0; s < P::kSub; ++s) {
                tma_load_4d(sbase + P::kA0 + s * P::kTile, &map_k, bar(P::bAFull), s * 64, c[1], c[2], c[3]);
                tma_load_4d(sbase + P::kA1 + s * P::kTile, &map_v, bar(P::bAFull), s * 64, c2[1], c2[2], c2[3]);
            }
            for (; issued < nitems && issued < P::kStages; ++issued) load_item(issued);
        }
    }
    if (warp == 8) tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // Everything below may read what the previous kernel in the stream wrote (delta, the
    // zeroed tickets): wait for it here (programmatic dependent launch).
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    mark(tp, 4);   // set-up done
    // S^T buffers at columns 0 and (D 64 only) 384; dP^T 128; dV 256; dK 256 + D.
    constexpr int kSBufs = 256 + 2 * D + 128 <= kTmemCols ? 2 : 1;
    const uint32_t tmem_dp = tmem + 128, tmem_dv = tmem + 256, tmem_dk = tmem + 256 + D;
    auto tmem_s_of = [&](int it) { return tmem + ((kSBufs == 2 && (it & 1)) ? 384u : 0u); };

    if (warp == 9) {
        // ---------------- producer ----------------
        if (nitems > 0) {
            for (int it = issued; it < nitems; ++it) {
                const int st = it % P::kStages;
                if (!__all_sync(0xffffffffu, mbar_wait(bar(P::bBEmpty + st), ((it / P::kStages) - 1) & 1, abort_flag, 400 + st, tp.status))) break;
                load_item(it);
                ++issued;
            }
            if (*abort_flag) {
                for (int it = max(0, issued - P::kStages); it < issued; ++it) {
                    const int st = it % P::kStages;
                    const long long t0 = clock64();
                    while (!mbar_try_wait(bar(P::bBFull + st), (it / P::kStages) & 1) && clock64() - t0 < kWaitCycles / 8) {
                    }
                }
            }
        }
    } else if (warp == 8) {
        // ---------------- MMA issuer ----------------
        if (nitems > 0) {
            constexpr uint32_t idesc_s = instr_desc(kBN, false);  // 128 x 128, both K-major
            constexpr uint32_t idesc_g = instr_desc(D, true);     // 128 x D, B MN-major
            const uint64_t k_desc = smem_desc(sbase + P::kA0, 16, 1024);
            const uint64_t v_desc = smem_desc(sbase + P::kA1, 16, 1024);
            const uint64_t q_desc = smem_desc(sbase + P::kB0, 16, 1024);
            const uint64_t do_desc = smem_desc(sbase + P::kB1, 16, 1024);
            const uint64_t q_mn = smem_desc(sbase + P::kB0, P::kTile, 1024);
            const uint64_t do_mn = smem_desc(sbase + P::kB1, P::kTile, 1024);
            bool ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bAFull), 0, abort_flag, 500, tp.status));
            if (ok && p.key_lengths && si.klen - k0 < kBM) {
                // Cache rows past the length may hold anything (0 x inf would poison dK and dV):
                // blank this CTA's key and value rows past it; their scores are masked anyway.
                const int first = si.klen - k0;   // > 0 here (nitems > 0)
                for (int idx = lane; idx < P::kSub * (kBM - first) * 8; idx += 32) {
                    const int sub = idx / ((kBM - first) * 8), rem = idx % ((kBM - first) * 8);
                    const int off = sub * P::kTile + (first + rem / 8) * 128 + (rem % 8) * 16;
                    *reinterpret_cast<uint4*>(smem + P::kA0 + off) = make_uint4(0u, 0u, 0u, 0u);
                    *reinterpret_cast<uint4*>(smem + P::kA1 + off) = make_uint4(0u, 0u, 0u, 0u);
                }
                fence_async_smem();
                __syncwarp();
            }
            // S^T = K Q^T of item `it` into its score buffer (the previous reader of that
            // buffer, dV of an earlier item, was issued before: MMAs run in issue order).
            auto issue_s = [&](int it) -> bool {
                const int st = it % P::kStages;
                const uint32_t soff = (st * P::kSub * P::kTile) >> 4;
                if (!__all_sync(0xffffffffu, mbar_wait(bar(P::bBFull + st), (it / P::kStages) & 1, abort_flag, 510 + st, tp.status))) return false;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t off = ((ks / 4) * P::kTile + (ks % 4) * 32) >> 4;
                    tc_mma(tmem_s_of(it), k_desc + off, q_desc + soff + off, idesc_s, ks > 0);
                }
                tc_commit(bar(P::bSReady + it % kSBufs));
                return true;
            };
            if (ok) ok = issue_s(0);
            for (int it = 0; ok && it < nitems; ++it) {
                const int st = it % P::kStages;
                const uint32_t soff = (st * P::kSub * P::kTile) >> 4;
                // dP^T = V dO^T, behind the previous item's dK (which read dS^T from there).
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t off = ((ks / 4) * P::kTile + (ks % 4) * 32) >> 4;
                    tc_mma(tmem_dp, v_desc + off, do_desc + soff + off, idesc_s, ks > 0);
                }
                tc_commit(bar(P::bDPReady));
                if (kSBufs == 2 && it + 1 < nitems) {
                    ok = issue_s(it + 1);
                    if (!ok) break;
                }
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bPFull + g), it & 1, abort_flag, 520 + g, tp.status));
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        // 16 query rows of this half per step: A = P^T / dS^T (8 TMEM columns),
                        // B = dO / Q rows as the MN-major operand (16 rows of 128 bytes).
                        const uint32_t boff = soff + (((g * 4 + ks) * 2048) >> 4);
                        const uint32_t acc = (it > 0 || g > 0 || ks > 0) ? 1u : 0u;
                        tc_mma_ts(tmem_dv, tmem_s_of(it) + g * 64 + ks * 8, do_mn + boff, idesc_g, acc);
                        tc_mma_ts(tmem_dk, tmem_dp + g * 64 + ks * 8, q_mn + boff, idesc_g, acc);
                    }
                }
                if (!ok) break;
                tc_commit(bar(P::bBEmpty + st));
                if (it + 1 == nitems) tc_commit(bar(P::bDone));
                if (kSBufs == 1 && it + 1 < nitems) ok = issue_s(it + 1);
            }
        }
    } else {
        // ---------------- score threads: (key row, half of the query columns) ----------------
        const int g = warp >> 2;
        const int row = (warp & 3) * 32 + lane;      // key inside the tile = TMEM lane
        const int kk = k0 + row;                     // key inside the sequence
        const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const bool key_ok = kk < si.klen;
        bool ok = true;
        uint32_t meets = 0;
        // The eight score warps meet (bounded: a warp that gave up cannot strand the others).
        auto meet = [&](int code) -> bool {
            mbar_arrive_warp(bar(P::bMeet));
            const bool met = __all_sync(0xffffffffu, mbar_wait(bar(P::bMeet), meets & 1, abort_flag, code, tp.status));
            ++meets;
            return met;
        };
        // A mask of one row per (batch, head): this thread's key has one term per query head.
        float mterm = 0.f;
        int cur_head = 0, cur_qb = 0;   // the item at hand: head inside this CTA's part, query block from qstart
        auto mask_term = [&](int) {
            if constexpr (kMask) {
                if (cur_qb == 0) {
                    const int h = hk * full_group + g0 + cur_head;
                    const int key = max(min(kk, si.klen - 1), 0);
                    mterm = mask_value(p, b, h, 0, static_cast<int64_t>(si.k_off) + key) * kLog2e;
                }
            }
        };

        // Row terms of one item: group 0 threads fetch lse, group 1 threads fetch delta. The
        // load is issued one item ahead and nothing looks at the loaded value until the next
        // item starts (a select or a multiply right behind the load would make the warp sit
        // out a trip to L2 in every item: measured, ~900 clk of a 3,300-clk item).
        // (Head and query block of the item to fetch are kept as running counters and the row's
        // address as a running pointer: the divisions and 64-bit products they replace were a
        // fifth of an item, one dependent chain per warp with nothing to overlap it.)
        int nxt_head = 0, nxt_qb = 0;   // item to fetch next: head inside this CTA's part, query block from qstart
        const float* src_row = g == 0
            ? p.lse + b * p.ls[0] + (hk * full_group + g0) * p.ls[1] + static_cast<int64_t>(si.q_off) * p.ls[2]
            : p.delta + b * p.delta_bs + (hk * full_group + g0) * p.delta_hs + si.q_off;
        const int64_t src_head = g == 0 ? p.ls[1] : p.delta_hs, src_step = g == 0 ? p.ls[2] : 1;
        auto fetch = [&](bool& exists) -> float {
            const int qi = (qstart + nxt_qb) * kBN + row;
            exists = qi < si.lq;
            const int qc = exists ? qi : 0;   // a row of this sequence, read and discarded
            const float raw = src_row[nxt_head * src_head + qc * src_step];
            if (++nxt_qb == per_head) {
                nxt_qb = 0;
                ++nxt_head;
            }
            return raw;
        };
        // What goes into the vectors: minus lse as base-2, ready to be added to the scaled
        // score (-inf for rows that do not exist or saw no key: P exactly 0), and delta (0 for
        // rows that do not exist).
        auto row_term = [&](float raw, bool exists) -> float {
            if (g == 0) {
                const float l = raw * kLog2e;
                return (!exists || l == -INFINITY) ? -INFINITY : -l;
            }
            return exists ? raw : 0.f;
        };
        // The vectors have three buffers (item mod 3) so that a warp can publish the terms of
        // item i + 1 and sign in at that item's meeting while it starts on item i: the buffer
        // it overwrites was read in item i - 2, which every warp has left (all have signed
        // in at meeting i, which they do at the top of item i - 1). By the time a warp
        // waits for meeting i + 1 the others have usually long signed in; met right after
        // the write, the warps waited for the slowest of them in every item (560 clk of a
        // 2,750-clk item).
        auto publish = [&](int it, float raw, bool exists) {
            float* buf = vec + (it % 3) * 256;
            (g == 0 ? buf : buf + 128)[row] = row_term(raw, exists);
            mbar_arrive_warp(bar(P::bMeet));
        };
        auto met_for = [&](int code) -> bool {
            const bool met = __all_sync(0xffffffffu, mbar_wait(bar(P::bMeet), meets & 1, abort_flag, code, tp.status));
            ++meets;
            return met;
        };
        bool pre_exists = false;
        float pre = 0.f;
        if (nitems > 0) {
            pre = fetch(pre_exists);
            publish(0, pre, pre_exists);
            if (nitems > 1) pre = fetch(pre_exists);
        }
        // While a trace buffer is set the CTA's first thread adds up where its item loop
        // waits (row 64 + 512 + CTA: meeting, wait for S, phase 1, wait for dP, phase 2).
        const bool timing = tp.trace && (threadIdx.x & 31) == 0 && blockIdx.x < 56;   // one row of 8 slots per warp
        long long acc_t[5] = {0, 0, 0, 0, 0}, tick = timing ? clock64() : 0;
        auto lap = [&](int slot) {
            if (timing) {
                const long long now = clock64();
                acc_t[slot] += now - tick;
                tick = now;
            }
        };

        for (int it = 0; it < nitems; ++it) {
            float* lse2 = vec + (it % 3) * 256;
            float* delta = lse2 + 128;
            ok = met_for(630);   // everybody's terms of item `it` are in
            if (!ok) break;
            if (it + 1 < nitems) publish(it + 1, pre, pre_exists);
            mask_term(it);
            if (it + 2 < nitems) pre = fetch(pre_exists);
            lap(0);
            const int q0 = (qstart + cur_qb) * kBN;
            const uint32_t tmem_s = tmem_s_of(it);
            ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bSReady + it % kSBufs), (it / kSBufs) & 1, abort_flag, 600 + g, tp.status));
            if (!ok) break;
            tc_fence_after();
            lap(1);
            if (it == 0) mark(tp, 5);   // first scores
            // Column c of this half is query q0 + g * 64 + c; key kk sees it when
            // kk <= q + shift, i.e. c >= first_col.
            const int first_col = p.causal ? kk - si.shift - q0 - g * 64 : -1;
            // Phase 1: P^T = 2^(S^T scale - lse), kept in registers and stored (bf16) over the
            // scores as the operand of dV. Two values per instruction on the packed fp32 pipe;
            // a tile every key of which sees every query of this half skips the tests.
            const bool whole = key_ok && first_col <= 0;
            const bool whole_w = __all_sync(0xffffffffu, whole);
            const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
            float2 pv[32];
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                float sc[32];
                tmem_ld32(tmem_s + lane_addr + g * 64 + c * 32, sc);
                tmem_wait_ld();
                const float4* l4 = reinterpret_cast<const float4*>(lse2 + g * 64 + c * 32);
                if (whole_w) {
                    // Every thread of the warp sees all its columns: no tests, and some pairs
                    // of every 8 as a cubic on the FMA pipe (with two score warps per
                    // scheduler the loop is bound by MUFU).
#pragma unroll
                    for (int e4 = 0; e4 < 8; ++e4) {
                        const float4 lv = l4[e4];
                        const float2 x0 = __ffma2_rn(make_float2(sc[e4 * 4], sc[e4 * 4 + 1]), sc2, (kMask ? make_float2(mterm + lv.x, mterm + lv.y) : make_float2(lv.x, lv.y)));
                        const float2 x1 = __ffma2_rn(make_float2(sc[e4 * 4 + 2], sc[e4 * 4 + 3]), sc2, (kMask ? make_float2(mterm + lv.z, mterm + lv.w) : make_float2(lv.z, lv.w)));
                        pv[c * 16 + e4 * 2] = poly_pair(e4 * 2) ? exp2_poly2_zero(x0) : make_float2(fast_exp2(x0.x), fast_exp2(x0.y));
                        pv[c * 16 + e4 * 2 + 1] = poly_pair(e4 * 2 + 1) ? exp2_poly2_zero(x1) : make_float2(fast_exp2(x1.x), fast_exp2(x1.y));
                    }
                } else {
#pragma unroll
                    for (int e4 = 0; e4 < 8; ++e4) {
                        const float4 lv = l4[e4];
                        float2 x0 = __ffma2_rn(make_float2(sc[e4 * 4], sc[e4 * 4 + 1]), sc2, (kMask ? make_float2(mterm + lv.x, mterm + lv.y) : make_float2(lv.x, lv.y)));
                        float2 x1 = __ffma2_rn(make_float2(sc[e4 * 4 + 2], sc[e4 * 4 + 3]), sc2, (kMask ? make_float2(mterm + lv.z, mterm + lv.w) : make_float2(lv.z, lv.w)));
                        if (!whole) {
                            const int col = c * 32 + e4 * 4;
                            x0.x = (key_ok && col >= first_col) ? x0.x : -INFINITY;
                            x0.y = (key_ok && col + 1 >= first_col) ? x0.y : -INFINITY;
                            x1.x = (key_ok && col + 2 >= first_col) ? x1.x : -INFINITY;
                            x1.y = (key_ok && col + 3 >= first_col) ? x1.y : -INFINITY;
                        }
                        // Hidden columns take MUFU, whose 2^-inf is exactly 0.
                        pv[c * 16 + e4 * 2] = make_float2(fast_exp2(x0.x), fast_exp2(x0.y));
                        pv[c * 16 + e4 * 2 + 1] = make_float2(fast_exp2(x1.x), fast_exp2(x1.y));
                    }
                }
            }
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t wp[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) wp[e] = pack_bf16(pv[c * 16 + e].x, pv[c * 16 + e].y);
                // Packed results go over columns this thread has already consumed.
                tmem_st16(tmem_s + lane_addr + g * 64 + c * 16, wp);
            }
            // Phase 2: dS^T = P^T o (dP^T - delta) over dP^T.
            lap(2);
            ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bDPReady), it & 1, abort_flag, 620 + g, tp.status));
            if (!ok) break;
            tc_fence_after();
            lap(3);
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                float dp[32];
                tmem_ld32(tmem_dp + lane_addr + g * 64 + c * 32, dp);
                tmem_wait_ld();
                uint32_t wd[16];
                const float4* d4 = reinterpret_cast<const float4*>(delta + g * 64 + c * 32);
#pragma unroll
                for (int e4 = 0; e4 < 8; ++e4) {
                    const float4 dv = d4[e4];
                    const float2 a0 = __fmul2_rn(pv[c * 16 + e4 * 2], __fadd2_rn(make_float2(dp[e4 * 4], dp[e4 * 4 + 1]), make_float2(-dv.x, -dv.y)));
                    const float2 a1 = __fmul2_rn(pv[c * 16 + e4 * 2 + 1], __fadd2_rn(make_float2(dp[e4 * 4 + 2], dp[e4 * 4 + 3]), make_float2(-dv.z, -dv.w)));
                    wd[e4 * 2] = pack_bf16(a0.x, a0.y);
                    wd[e4 * 2 + 1] = pack_bf16(a1.x, a1.y);
                }
                tmem_st16(tmem_dp + lane_addr + g * 64 + c * 16, wd);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive_warp(bar(P::bPFull + g));
            if (++cur_qb == per_head) {
                cur_qb = 0;
                ++cur_head;
            }
            lap(4);
        }
        if (timing) {
            long long* out = tp.trace + (64 + 512 + blockIdx.x * 8 + warp) * 8;
            for (int i = 0; i < 5; ++i) out[i] = acc_t[i];
            out[5] = nitems;
        }

        // Epilogue: group 0 writes dV, group 1 writes dK (scaled); rows past the end of the
        // sequence are not stored. Every lane takes part in the TMEM reads. With the GQA
        // group split over several CTAs the fp32 sums go to the partial buffer instead.
        if (ok && nitems > 0) ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bDone), 0, abort_flag, 610, tp.status));
        mark(tp, 6);   // last MMA done
        if (ok) {
            const bool real = kk < si.lk;
            const float mul = g == 0 ? 1.f : p.scale;
            __nv_bfloat16* dst = g == 0
                ? p.dv_out + b * p.dvs[0] + hk * p.dvs[1] + static_cast<int64_t>(si.k_off + kk) * p.dvs[2]
                : p.dk + b * p.dks[0] + hk * p.dks[1] + static_cast<int64_t>(si.k_off + kk) * p.dks[2];
            const int64_t key_rows = p.cu_q ? p.total_k : p.sk;
            const int64_t planes = static_cast<int64_t>(p.cu_q ? 1 : p.batch) * p.kv_heads * p.gsplit;
            // A part's partial block is stored column-major in float4 units ([D / 4][rows of the
            // block that exist]): a warp's store then covers 512 contiguous bytes where a
            // thread-per-row layout touched 32 sectors at a stride of a row (measured: 2.0 of
            // the 2.5 us a dK/dV CTA spent storing its results).
            const int block_rows = min(kBM, si.lk - k0);
            float4* pdst = reinterpret_cast<float4*>(
                p.dkv_partial + (g * planes + (static_cast<int64_t>(p.cu_q ? 0 : b) * p.kv_heads + hk) * p.gsplit + part) * key_rows * D +
                static_cast<int64_t>(si.k_off + k0) * D) + row;
            if (nitems > 0) tc_fence_after();
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                float o[32];
                if (nitems > 0) {
                    tmem_ld32((g == 0 ? tmem_dv : tmem_dk) + lane_addr + c * 32, o);
                    tmem_wait_ld();
                } else {
#pragma unroll
                    for (int e = 0; e < 32; ++e) o[e] = 0.f;
                }
                if (real && p.gsplit > 1) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        pdst[(c * 8 + e) * block_rows] = make_float4(o[e * 4], o[e * 4 + 1], o[e * 4 + 2], o[e * 4 + 3]);
                    }
                } else if (real) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        uint32_t w[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) w[i] = pack_bf16(o[e * 16 + 2 * i] * mul, o[e * 16 + 2 * i + 1] * mul);
                        store_32_bytes(dst + c * 32 + e * 16, w);
                    }
                }
            }
        }
        mark(tp, 7);   // own results stored
        if (p.gsplit > 1 && p.dkv_counters) {
            // The CTAs sharing this key block take a ticket each once their partial is
            // stored; the one that draws the last sums the partials in the order of the
            // parts (deterministic, the same sums whoever is last) and writes bf16.
            // Every score thread comes here, whatever its waits returned.
            int* last_flag = reinterpret_cast<int*>(vec);
            bool met = meet(640);  // all partial stores of this CTA are done
            if (threadIdx.x == 0) {
                int ticket = 0;
                if (ok) {
                    int32_t* counter = p.dkv_counters + (static_cast<int64_t>(b) * p.kv_heads + hk) * gridDim_y + kb;
                    asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(ticket) : "l"(counter) : "memory");
                }
                *last_flag = ok && ticket == p.gsplit - 1;
            }
            met = meet(641) && met;
            if (met && *last_flag) {
                // The 128 threads of a group sum their plane (dV or dK) of the key block, thread
                // r the row r: the parts are column-major in float4 units (see the stores
                // above), so a warp reads 512 contiguous bytes per part and position. All parts
                // of two positions are requested before any is used (the sums wait for L2 once
                // per two positions, not once per part), and are added in the order of the
                // parts: the same bits whoever is last.
                const float mul = g == 0 ? 1.f : p.scale;
                const int block_rows = min(kBM, si.lk - k0);
                __nv_bfloat16* dst = (g == 0 ? p.dv_out + b * p.dvs[0] + hk * p.dvs[1] : p.dk + b * p.dks[0] + hk * p.dks[1]) +
                                     static_cast<int64_t>(si.k_off + k0 + row) * (g == 0 ? p.dvs[2] : p.dks[2]);
                const int64_t key_rows = p.cu_q ? p.total_k : p.sk;
                const int64_t planes = static_cast<int64_t>(p.cu_q ? 1 : p.batch) * p.kv_heads * p.gsplit;
                const float* src = p.dkv_partial + (g * planes + (static_cast<int64_t>(p.cu_q ? 0 : b) * p.kv_heads + hk) * p.gsplit) * key_rows * D +
                                   static_cast<int64_t>(si.k_off + k0) * D;
                const int64_t part_stride = key_rows * D;
                constexpr int kPositions = D / 4;   // float4 positions per thread: the row's columns
                constexpr int kMaxParts = 8;        // backward_group_split never asks for more
                if (row < block_rows) {
                    for (int i = 0; i < kPositions; i += 2) {
                        float4 part[2][kMaxParts];
#pragma unroll
                        for (int u = 0; u < 2; ++u) {
#pragma unroll
                            for (int s_ = 0; s_ < kMaxParts; ++s_) {
                                if (s_ < p.gsplit) part[u][s_] = __ldcg(reinterpret_cast<const float4*>(src + s_ * part_stride) + (i + u) * block_rows + row);
                            }
                        }
#pragma unroll
                        for (int u = 0; u < 2; ++u) {
                            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                            for (int s_ = 0; s_ < kMaxParts; ++s_) {
                                if (s_ < p.gsplit) {
                                    acc.x += part[u][s_].x;
                                    acc.y += part[u][s_].y;
                                    acc.z += part[u][s_].z;
                                    acc.w += part[u][s_].w;
                                }
                            }
                            uint2 v;
                            v.x = pack_bf16(acc.x * mul, acc.y * mul);
                            v.y = pack_bf16(acc.z * mul, acc.w * mul);
                            *reinterpret_cast<uint2*>(dst + (i + u) * 4) = v;
                        }
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        if (*abort_flag) {
            const long long t0 = clock64();
            while (clock64() - t0 < 2000000) {
            }
        }
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

// ---- dQ ---------------------------------------------------------------------------------

// Body of one dQ CTA; (bx, by, bz) = (head, query block counted from the end, batch).
template <int D, bool kMask>
__device__ __forceinline__ void dq_body(
    const CUtensorMap* pmap_q, const CUtensorMap* pmap_k, const CUtensorMap* pmap_v, const CUtensorMap* pmap_do,
    const BwdParams& tp, int bx, int by, int bz, int ny) {
    const CUtensorMap& map_q = *pmap_q;
    const CUtensorMap& map_k = *pmap_k;
    const CUtensorMap& map_v = *pmap_v;
    const CUtensorMap& map_do = *pmap_do;
    using P = BwdPlan<D>;
    extern __shared__ __align__(1024) unsigned char smem[];
    const uint32_t sbase = smem_u32(smem);
    if (sbase & 1023u) {
        if (threadIdx.x == 0) atomicCAS_system(tp.status, 0, 902);
        return;
    }
    const uint32_t bars = sbase + P::kBars;
    auto bar = [&](int i) { return bars + 8u * i; };
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + P::kBars + P::bCount * 8);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + P::kBars + P::bCount * 8 + 8);

    const AttnParams& p = tp.a;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = bx, b = bz;
    const int qb = ny - 1 - by;
    const SeqInfo si = seq_info(p, b);
    const int q0 = qb * kBM;
    if (q0 >= si.lq) return;
    const int hk = div_by(h, tp.by_group);
    int kend = si.klen;
    if (p.causal) kend = min(kend, min(q0 + kBM, si.lq) - 1 + si.shift + 1);
    const int nblocks = kend > 0 ? (kend + kBN - 1) / kBN : 0;

    auto coords = [&](int operand, int row, int head, int batch, int (&c)[4]) {
        c[tp.dim_of[operand][0]] = row;
        c[tp.dim_of[operand][1]] = head;
        c[tp.dim_of[operand][2]] = batch;
    };
    const int batch_c = p.cu_q ? 0 : b;
    // K and V tiles of key block j into their ring stage (producer warp, converged).
    auto load_block = [&](int j) {
        int c[4], c2[4];
        c[0] = c2[0] = 0;
        const int st = j % P::kStages;
        coords(1, si.k_off + j * kBN, hk, batch_c, c);
        coords(2, si.k_off + j * kBN, hk, batch_c, c2);
        mbar_expect_tx(bar(P::bBFull + st), 2 * P::kSub * P::kTile);
        for (int s = 0; s < P::kSub; ++s) {
            tma_load_4d(sbase + P::kB0 + (st * P::kSub + s) * P::kTile, &map_k, bar(P::bBFull + st), s * 64, c[1], c[2], c[3]);
            tma_load_4d(sbase + P::kB1 + (st * P::kSub + s) * P::kTile, &map_v, bar(P::bBFull + st), s * 64, c2[1], c2[2], c2[3]);
        }
    };

    // Set-up as in the dK/dV body: the producer warp initialises the barriers and sends the
    // first loads while tensor memory is being allocated.
    int issued = 0;
    if (warp == 9) {
        if (lane == 0) init_barriers<D>(bars, abort_flag);
        __syncwarp();
        if (nblocks > 0) {
            int c[4], c2[4];
            c[0] = c2[0] = 0;
            coords(0, si.q_off + q0, h, batch_c, c);
            coords(3, si.q_off + q0, h, batch_c, c2);
            mbar_expect_tx(bar(P::bAFull), 2 * P::kSub * P::kTile);
            for (int s = 0; s < P::kSub; ++s) {
                tma_load_4d(sbase + P::kA0 + s * P::kTile, &map_q, bar(P::bAFull), s * 64, c[1], c[2], c[3]);
                tma_load_4d(sbase + P::kA1 + s * P::kTile, &map_do, bar(P::bAFull), s * 64, c2[1], c2[2], c2[3]);
            }
            for (; issued < nblocks && issued < P::kStages; ++issued) load_block(issued);
        }
    }
    if (warp == 8) tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    asm volatile("griddepcontrol.wait;" ::: "memory");   // delta comes from the previous kernel in the stream
    const uint32_t tmem = *tmem_slot;
    mark(tp, 4);
    // S buffers at columns 0 and 384, dP 128, dQ 256 (D <= 128 columns).
    const uint32_t tmem_dp = tmem + 128, tmem_dq = tmem + 256;
    auto tmem_s_of = [&](int j) { return tmem + ((j & 1) ? 384u : 0u); };

    if (warp == 9) {
        if (nblocks > 0) {
            for (int j = issued; j < nblocks; ++j) {
                const int st = j % P::kStages;
                if (!__all_sync(0xffffffffu, mbar_wait(bar(P::bBEmpty + st), ((j / P::kStages) - 1) & 1, abort_flag, 700 + st, tp.status))) break;
                load_block(j);
                ++issued;
            }
            if (*abort_flag) {
                for (int j = max(0, issued - P::kStages); j < issued; ++j) {
                    const int st = j % P::kStages;
                    const long long t0 = clock64();
                    while (!mbar_try_wait(bar(P::bBFull + st), (j / P::kStages) & 1) && clock64() - t0 < kWaitCycles / 8) {
                    }
                }
            }
        }
    } else if (warp == 8) {
        if (nblocks > 0) {
            constexpr uint32_t idesc_s = instr_desc(kBN, false);
            constexpr uint32_t idesc_g = instr_desc(D, true);
            const uint64_t q_desc = smem_desc(sbase + P::kA0, 16, 1024);
            const uint64_t do_desc = smem_desc(sbase + P::kA1, 16, 1024);
            const uint64_t k_desc = smem_desc(sbase + P::kB0, 16, 1024);
            const uint64_t v_desc = smem_desc(sbase + P::kB1, 16, 1024);
            const uint64_t k_mn = smem_desc(sbase + P::kB0, P::kTile, 1024);
            bool ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bAFull), 0, abort_flag, 800, tp.status));
            // S = Q K^T of block j into its buffer: free since the threads published dS of
            // block j - 2 (they only read the scores).
            auto issue_s = [&](int j) -> bool {
                const int st = j % P::kStages;
                const uint32_t soff = (st * P::kSub * P::kTile) >> 4;
                if (!__all_sync(0xffffffffu, mbar_wait(bar(P::bBFull + st), (j / P::kStages) & 1, abort_flag, 810 + st, tp.status))) return false;
                if (p.key_lengths && si.klen - j * kBN < kBN) {
                    // Blank the key and value rows past the length (see the dK/dV body).
                    const int first = si.klen - j * kBN;   // > 0: the block has a visible key
                    for (int idx = lane; idx < P::kSub * (kBN - first) * 8; idx += 32) {
                        const int sub = idx / ((kBN - first) * 8), rem = idx % ((kBN - first) * 8);
                        const int off = (st * P::kSub + sub) * P::kTile + (first + rem / 8) * 128 + (rem % 8) * 16;
                        *reinterpret_cast<uint4*>(smem + P::kB0 + off) = make_uint4(0u, 0u, 0u, 0u);
                        *reinterpret_cast<uint4*>(smem + P::kB1 + off) = make_uint4(0u, 0u, 0u, 0u);
                    }
                    fence_async_smem();
                    __syncwarp();
                }
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t off = ((ks / 4) * P::kTile + (ks % 4) * 32) >> 4;
                    tc_mma(tmem_s_of(j), q_desc + off, k_desc + soff + off, idesc_s, ks > 0);
                }
                tc_commit(bar(P::bSReady + (j & 1)));
                return true;
            };
            if (ok) ok = issue_s(0);
            for (int j = 0; ok && j < nblocks; ++j) {
                const int st = j % P::kStages;
                const uint32_t soff = (st * P::kSub * P::kTile) >> 4;
                // dP = dO V^T, behind the previous block's dQ MMA (which read dS from there).
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t off = ((ks / 4) * P::kTile + (ks % 4) * 32) >> 4;
                    tc_mma(tmem_dp, do_desc + off, v_desc + soff + off, idesc_s, ks > 0);
                }
                tc_commit(bar(P::bDPReady));
                if (j + 1 < nblocks) {
                    ok = issue_s(j + 1);
                    if (!ok) break;
                }
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bPFull + g), j & 1, abort_flag, 820 + g, tp.status));
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        tc_mma_ts(tmem_dq, tmem_dp + g * 64 + ks * 8,
                                  k_mn + soff + (((g * 4 + ks) * 2048) >> 4), idesc_g, (j > 0 || g > 0 || ks > 0) ? 1u : 0u);
                    }
                }
                if (!ok) break;
                tc_commit(bar(P::bBEmpty + st));
                if (j + 1 == nblocks) tc_commit(bar(P::bDone));
            }
        }
    } else {
        // ---------------- score threads: (query row, half of the key columns) ----------------
        const int g = warp >> 2;
        const int row = (warp & 3) * 32 + lane;
        const int qi = q0 + row;
        const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
        bool ok = true;
        float lse2 = INFINITY, delta = 0.f;
        if (qi < si.lq) {
            lse2 = p.lse[b * p.ls[0] + h * p.ls[1] + (si.q_off + qi) * p.ls[2]] * kLog2e;
            if (lse2 == -INFINITY) lse2 = INFINITY;  // a row without keys: P exactly 0
            delta = p.delta[b * p.delta_bs + h * p.delta_hs + si.q_off + qi];
        }
        int row_limit = si.klen;
        if (p.causal) row_limit = min(row_limit, qi + si.shift + 1);
        float* vec = reinterpret_cast<float*>(smem + P::kVec);   // [block parity][128]: a block's mask terms
        // Item-loop clocks per score warp while a trace buffer is set, as in the dK/dV body
        // (rows 64 + 512 + 448 + 8 (CTA - first dQ CTA) + warp; first 8 dQ CTAs).
        const int dq_index = static_cast<int>(blockIdx.x) - static_cast<int>(gridDim.x - static_cast<unsigned>(p.heads) * ny * p.batch);
        const bool timing = tp.trace && lane == 0 && dq_index >= 0 && dq_index < 8;
        long long acc_t[5] = {0, 0, 0, 0, 0}, tick = timing ? clock64() : 0;
        auto lap = [&](int slot) {
            if (timing) {
                const long long now = clock64();
                acc_t[slot] += now - tick;
                tick = now;
            }
        };

        for (int j = 0; j < nblocks; ++j) {
            if constexpr (kMask) {
                // A mask of one row per (batch, head): one thread per key column fetches the
                // block's terms; the buffer of block j - 2 is free (everybody met since).
                if (g == 0) {
                    const int key = max(min(j * kBN + row, si.klen - 1), 0);
                    vec[(j & 1) * 128 + row] = mask_value(p, b, h, 0, static_cast<int64_t>(si.k_off) + key) * kLog2e;
                }
                mbar_arrive_warp(bar(P::bMeet));
                ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bMeet), j & 1, abort_flag, 930 + g, tp.status));
                if (!ok) break;
            }
            lap(0);
            ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bSReady + (j & 1)), (j >> 1) & 1, abort_flag, 900 + g, tp.status));
            if (!ok) break;
            tc_fence_after();
            lap(1);
            if (j == 0) mark(tp, 5);
            const int limit = row_limit - j * kBN - g * 64;  // this half's columns [0, limit) are visible
            // Phase 1: P in registers while dP of this block is still being computed. Two
            // values per instruction on the packed fp32 pipe; wholly visible halves skip the
            // tests.
            const bool whole = limit >= 64;
            const bool whole_w = __all_sync(0xffffffffu, whole);
            const float2 sc2 = make_float2(p.scale_log2, p.scale_log2), nl2 = make_float2(-lse2, -lse2);
            const float2 nd2 = make_float2(-delta, -delta);
            float2 pv[32];
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                float sc[32];
                tmem_ld32(tmem_s_of(j) + lane_addr + g * 64 + c * 32, sc);
                tmem_wait_ld();
                if (whole_w) {
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        float2 x = __ffma2_rn(make_float2(sc[2 * e], sc[2 * e + 1]), sc2, nl2);
                        if constexpr (kMask) {
                            const float2 t = reinterpret_cast<const float2*>(vec + (j & 1) * 128 + g * 64 + c * 32)[e];
                            x = __fadd2_rn(x, t);
                        }
                        pv[c * 16 + e] = poly_pair(e) ? exp2_poly2_zero(x) : make_float2(fast_exp2(x.x), fast_exp2(x.y));
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        float2 x = __ffma2_rn(make_float2(sc[2 * e], sc[2 * e + 1]), sc2, nl2);
                        if constexpr (kMask) {
                            const float2 t = reinterpret_cast<const float2*>(vec + (j & 1) * 128 + g * 64 + c * 32)[e];
                            x = __fadd2_rn(x, t);
                        }
                        if (!whole) {
                            x.x = c * 32 + 2 * e < limit ? x.x : -INFINITY;
                            x.y = c * 32 + 2 * e + 1 < limit ? x.y : -INFINITY;
                        }
                        pv[c * 16 + e] = make_float2(fast_exp2(x.x), fast_exp2(x.y));
                    }
                }
            }
            // Phase 2: dS = P o (dP - delta) over dP.
            lap(2);
            ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bDPReady), j & 1, abort_flag, 920 + g, tp.status));
            if (!ok) break;
            tc_fence_after();
            lap(3);
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                float dp[32];
                tmem_ld32(tmem_dp + lane_addr + g * 64 + c * 32, dp);
                tmem_wait_ld();
                uint32_t wd[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    float2 a = __fmul2_rn(pv[c * 16 + e], __fadd2_rn(make_float2(dp[2 * e], dp[2 * e + 1]), nd2));
                    if (!whole_w) {   // hidden keys: exactly 0 whatever dP holds there (a warp-wide test: no selects in whole tiles)
                        a.x = c * 32 + 2 * e < limit ? a.x : 0.f;
                        a.y = c * 32 + 2 * e + 1 < limit ? a.y : 0.f;
                    }
                    wd[e] = pack_bf16(a.x, a.y);
                }
                tmem_st16(tmem_dp + lane_addr + g * 64 + c * 16, wd);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive_warp(bar(P::bPFull + g));
            lap(4);
        }
        if (timing) {
            long long* out = tp.trace + (64 + 512 + 448 + dq_index * 8 + warp) * 8;
            for (int i = 0; i < 5; ++i) out[i] = acc_t[i];
            out[5] = nblocks;
        }

        if (ok && nblocks > 0) ok = __all_sync(0xffffffffu, mbar_wait(bar(P::bDone), 0, abort_flag, 910, tp.status));
        mark(tp, 6);
        if (ok) {
            // Group g writes dQ columns [g * D / 2, (g + 1) * D / 2), scaled.
            const bool real = qi < si.lq;
            __nv_bfloat16* dst = p.dq + b * p.dqs[0] + h * p.dqs[1] + static_cast<int64_t>(si.q_off + qi) * p.dqs[2] + g * (D / 2);
            if (nblocks > 0) tc_fence_after();
#pragma unroll
            for (int c = 0; c < D / 64; ++c) {
                float o[32];
                if (nblocks > 0) {
                    tmem_ld32(tmem_dq + lane_addr + g * (D / 2) + c * 32, o);
                    tmem_wait_ld();
                } else {
#pragma unroll
                    for (int e = 0; e < 32; ++e) o[e] = 0.f;
                }
                if (real) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        uint32_t w[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) w[i] = pack_bf16(o[e * 16 + 2 * i] * p.scale, o[e * 16 + 2 * i + 1] * p.scale);
                        store_32_bytes(dst + c * 32 + e * 16, w);
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        if (*abort_flag) {
            const long long t0 = clock64();
            while (clock64() - t0 < 2000000) {
            }
        }
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

// One launch for both halves of the backward: CTAs [0, n_dkv) are dK/dV CTAs, the rest dQ
// CTAs (each list longest first). The two are independent of each other, and in one grid the
// dQ CTAs fill the SMs that the tail of the dK/dV list leaves idle.
template <int D, bool kMask>
__global__ void __launch_bounds__(kThreads, 1) bwd_tc5_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
    const BwdParams tp, int dkv_x, int dkv_y, int n_dkv, int dq_x, int dq_y) {
    int id = blockIdx.x;
    long long t_start = 0;
    if (tp.trace && threadIdx.x == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_start));
    struct Stamp {   // while a trace buffer is set: start, end, SM and index of every CTA (rows 64 + CTA)
        const BwdParams& tp;
        long long t0;
        __device__ ~Stamp() {
            if (tp.trace && threadIdx.x == 0 && blockIdx.x < 1024) {
                long long t1;
                unsigned smid;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
                asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
                long long* out = tp.trace + (64 + blockIdx.x) * 8;
                out[0] = t0;
                out[1] = t1;
                out[2] = smid;
                out[3] = blockIdx.x;
            }
        }
    } stamp{tp, t_start};
    if (id < n_dkv) {
        const int rest = div_by(id, tp.by_dkv_x), bz = div_by(rest, tp.by_dkv_y);
        dkv_body<D, kMask>(&map_q, &map_k, &map_v, &map_do, tp, id - rest * dkv_x, rest - bz * dkv_y, bz, dkv_y);
    } else {
        id -= n_dkv;
        const int rest = div_by(id, tp.by_dq_x), bz = div_by(rest, tp.by_dq_y);
        dq_body<D, kMask>(&map_q, &map_k, &map_v, &map_do, tp, id - rest * dq_x, rest - bz * dq_y, bz, dq_y);
    }
}

bool aligned16(const void* ptr, const int64_t strides[3]) {
    if (reinterpret_cast<uintptr_t>(ptr) & 15) return false;
    for (int i = 0; i < 3; ++i) {
        if (strides[i] % 8) return false;
    }
    return true;
}

template <int D>
int launch_bwd(const AttnParams& p, cudaStream_t stream) {
    using P = BwdPlan<D>;
    const char* why = "";
    const int64_t tq = p.cu_q ? p.total_q : p.sq, tk = p.cu_q ? p.total_k : p.sk;
    const int64_t bq = p.cu_q ? 1 : p.batch;
    int64_t s[4][3];
    if (!operand_layout(p.q, tq, p.heads, bq, p.qs, s[0], &why) ||
        !operand_layout(p.k, tk, p.kv_heads, bq, p.ks, s[1], &why) ||
        !operand_layout(p.v, tk, p.kv_heads, bq, p.vs, s[2], &why) ||
        !operand_layout(p.dout, tq, p.heads, bq, p.dos, s[3], &why)) {
        return fail(KTT_B200_ERR_UNSUPPORTED, "tcgen05 backward: %s", why);
    }
    DimOrder orders[4];
    for (int i = 0; i < 4; ++i) orders[i] = order_of(s[i]);
    CUtensorMap mq, mk, mv, mdo;
    if (!encode_map(&mq, p.q, D, tq, p.heads, bq, s[0], orders[0], kBM, &why) ||
        !encode_map(&mk, p.k, D, tk, p.kv_heads, bq, s[1], orders[1], kBM, &why) ||
        !encode_map(&mv, p.v, D, tk, p.kv_heads, bq, s[2], orders[2], kBM, &why) ||
        !encode_map(&mdo, p.dout, D, tq, p.heads, bq, s[3], orders[3], kBM, &why)) {
        return fail(KTT_B200_ERR_UNSUPPORTED, "tcgen05 backward: %s", why);
    }
    BwdParams tp;
    tp.a = p;
    int* dev_status = nullptr;
    int* host_status = status_word(&dev_status);
    if (!host_status || !dev_status) return fail(KTT_B200_ERR_LAUNCH, "tcgen05 backward: no status word");
    if (*host_status != 0) {
        const int code = *host_status;
        *host_status = 0;
        note_call(5);
        return fail(KTT_B200_ERR_DEVICE_WAIT, "an earlier tcgen05 launch gave up waiting (code %d)", code);
    }
    tp.status = dev_status;
    tp.trace = tc5::trace_buffer();
    for (int o = 0; o < 4; ++o) {
        for (int i = 0; i < 3; ++i) tp.dim_of[o][i] = orders[o].slot_of[i];
    }
    constexpr int smem = P::kBytes;
    const bool masked = p.mask_dtype != KTT_B200_MASK_NONE;
    auto kernel = masked ? bwd_tc5_kernel<D, true> : bwd_tc5_kernel<D, false>;
    if (int rc = ensure_smem(kernel, smem, "cudaFuncSetAttribute(bwd_tc5)")) return rc;
    const int dkv_x = p.kv_heads * p.gsplit, dkv_y = (p.sk + kBM - 1) / kBM;
    const int dq_x = p.heads, dq_y = (p.sq + kBM - 1) / kBM;
    tp.by_dkv_x = divisor_of(dkv_x);
    tp.by_dkv_y = divisor_of(dkv_y > 0 ? dkv_y : 1);
    tp.by_dq_x = divisor_of(dq_x);
    tp.by_dq_y = divisor_of(dq_y > 0 ? dq_y : 1);
    tp.by_gsplit = divisor_of(p.gsplit);
    tp.by_group = divisor_of(p.heads / p.kv_heads);
    const int64_t n_dkv = static_cast<int64_t>(dkv_x) * dkv_y * p.batch;
    const int64_t n_all = n_dkv + static_cast<int64_t>(dq_x) * dq_y * p.batch;
    if (n_all > 0x7fffffff) return fail(KTT_B200_ERR_UNSUPPORTED, "tcgen05 backward: too many tiles");
    if (p.gsplit > 1 && !p.dkv_counters) return fail(KTT_B200_ERR_BAD_ARGUMENT, "tcgen05 backward: the group split needs its ticket counters");
    // Programmatic dependent launch behind the delta kernel: set-up and the first loads of
    // every CTA of the first wave run while that kernel drains.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(n_all));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return check_cuda(cudaLaunchKernelEx(&cfg, kernel, mq, mk, mv, mdo, tp, dkv_x, dkv_y, static_cast<int>(n_dkv), dq_x, dq_y),
                      "bwd_tc5 launch");
}

}  // namespace

bool backward_tc5_takes(const AttnParams& p, const char** why) {
    // Masks of one row per (batch, head) and key lengths are taken (forward_tc5_takes keeps
    // the masks that differ between query rows on the warp-MMA kernels).
    if (!forward_tc5_takes(p, why)) return false;
    if (!aligned16(p.dout, p.dos) || !aligned16(p.dq, p.dqs) || !aligned16(p.dk, p.dks) || !aligned16(p.dv_out, p.dvs)) {
        *why = "dout, dq, dk and dv must be 16-byte aligned with strides that are multiples of 8";
        return false;
    }
    return true;
}

int backward_group_split(const AttnParams& p) {
    const int group = p.heads / p.kv_heads;
    if (group <= 1 || p.d != p.dv || (p.d != 64 && p.d != 128)) return 1;
    // Aim for about 256 CTAs: the dK/dV kernel has one CTA per (batch, kv head, 128 keys).
    const int64_t ctas = static_cast<int64_t>(p.batch) * p.kv_heads * ((p.sk + kBM - 1) / kBM);
    const int64_t want = ctas > 0 ? 256 / ctas : 1;
    if (want <= 1) return 1;
    const int64_t cap = want < group ? want : group;
    return static_cast<int>(cap < 8 ? cap : 8);   // the ticketed sum holds at most 8 parts at a time
}

int64_t backward_counter_offset(const AttnParams& p, int gsplit) {
    if (gsplit <= 1) return 0;
    const int64_t key_rows = p.cu_q ? p.total_k : p.sk;
    const int64_t nb = p.cu_q ? 1 : p.batch;
    return (2 * nb * p.kv_heads * gsplit * key_rows * p.d * 4 + 255) / 256 * 256;
}

int64_t backward_counter_count(const AttnParams& p, int gsplit) {
    if (gsplit <= 1) return 0;
    return static_cast<int64_t>(p.batch) * p.kv_heads * ((p.sk + kBM - 1) / kBM);
}

int64_t backward_partial_bytes(const AttnParams& p, int gsplit) {
    if (gsplit <= 1) return 0;
    return backward_counter_offset(p, gsplit) + (backward_counter_count(p, gsplit) * 4 + 255) / 256 * 256;
}

int launch_backward_tc5(const AttnParams& p, cudaStream_t stream) {
    if (int rc = launch_backward_delta(p, stream)) return rc;
    if (p.d == 64) return launch_bwd<64>(p, stream);
    return launch_bwd<128>(p, stream);
}

}  // namespace ktt
