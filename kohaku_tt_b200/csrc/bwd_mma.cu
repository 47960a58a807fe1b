// General backward on warp-level MMA: row statistics, a dQ kernel and a dK/dV kernel.
//
// Same split as the reference's backward (ktt_flash/program.cpp:1587-2006: a dQ program
// that also produces the row terms, then a dK/dV program), so every gradient has one
// owner and the result is deterministic without atomics:
//   delta_i = sum_d dO_id O_id                          (ktt_flash/bw_dq_compute.cpp)
//   P_ij    = 2^(x_ij - lse_i log2e),  x = logits in base 2 (recomputed, never stored)
//   dP_ij   = dO_i . V_j
//   dS_ij   = P_ij (dP_ij - delta_i)
//   dQ_i    = scale * sum_j dS_ij K_j                   (one CTA per 64 query rows)
//   dV_j    = sum_i P_ij dO_i,  dK_j = scale * sum_i dS_ij Q_i
//                                   (one CTA per 64 keys, summed over the GQA group)
// Keys a row cannot see give P exactly 0, hence exactly zero gradients.
#include "tiles.cuh"

namespace ktt {
namespace {

constexpr int kThreads = 128;

// The first kernel of every backward also clears the tickets of the dK/dV CTAs that share a
// key block (a grid of the delta kernels always has more threads than there are counters).
__device__ __forceinline__ void zero_counters(int32_t* counters, int64_t n) {
    if (!counters) return;
    const int64_t block = (static_cast<int64_t>(blockIdx.z) * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
    const int64_t i = block * blockDim.x + threadIdx.x;
    if (i < n) counters[i] = 0;
}

// delta[b, h, i] = sum_d dO * O, one warp per row (any width and alignment).
__global__ void __launch_bounds__(kThreads) bwd_delta_kernel(const AttnParams p, int64_t ncounters) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    zero_counters(p.dkv_counters, ncounters);
    const int b = blockIdx.z, h = blockIdx.y;
    const SeqInfo si = seq_info(p, b);
    const int row = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
    if (row >= si.lq) return;
    const int lane = threadIdx.x & 31;
    const __nv_bfloat16* og = p.out + b * p.os[0] + h * p.os[1] + static_cast<int64_t>(si.q_off + row) * p.os[2];
    const __nv_bfloat16* dg = p.dout + b * p.dos[0] + h * p.dos[1] + static_cast<int64_t>(si.q_off + row) * p.dos[2];
    float acc = 0.f;
    for (int c = lane; c < p.dv; c += 32) {
        acc += __bfloat162float(og[c]) * __bfloat162float(dg[c]);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) p.delta[b * p.delta_bs + h * p.delta_hs + si.q_off + row] = acc;
}

// The same with 16-byte loads: LANES = Dv / 8 lanes per row, 256 / LANES rows per CTA.
// Needs Dv in {64, 128} and 16-byte aligned rows (the launcher checks).
template <int DV>
__global__ void __launch_bounds__(256) bwd_delta_vec_kernel(const AttnParams p, int64_t ncounters) {
    // The backward kernel behind this one may start its set-up and input loads now; it waits
    // (griddepcontrol.wait) for this kernel to finish before it reads delta or the tickets.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    zero_counters(p.dkv_counters, ncounters);
    constexpr int LANES = DV / 8, ROWS = 256 / LANES;
    const int b = blockIdx.z, h = blockIdx.y;
    const SeqInfo si = seq_info(p, b);
    const int row = blockIdx.x * ROWS + threadIdx.x / LANES;
    const int c = (threadIdx.x % LANES) * 8;
    float acc = 0.f;
    if (row < si.lq) {
        const uint4 o = __ldg(reinterpret_cast<const uint4*>(
            p.out + b * p.os[0] + h * p.os[1] + static_cast<int64_t>(si.q_off + row) * p.os[2] + c));
        const uint4 d = __ldg(reinterpret_cast<const uint4*>(
            p.dout + b * p.dos[0] + h * p.dos[1] + static_cast<int64_t>(si.q_off + row) * p.dos[2] + c));
        const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&o);
        const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&d);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 x = __bfloat1622float2(o2[e]), y = __bfloat1622float2(d2[e]);
            acc = fmaf(x.x, y.x, acc);
            acc = fmaf(x.y, y.y, acc);
        }
    }
#pragma unroll
    for (int off = LANES / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (row < si.lq && c == 0) p.delta[b * p.delta_bs + h * p.delta_hs + si.q_off + row] = acc;
}

// dQ: one CTA per (64 query rows, head, batch); streams key/value blocks.
template <int DP, int BN>
__global__ void __launch_bounds__(kThreads) bwd_dq_kernel(const AttnParams p) {
    constexpr int BM = 64;
    constexpr int LD = DP + kPad;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* sdO = sQ + BM * LD;
    __nv_bfloat16* sK = sdO + BM * LD;
    __nv_bfloat16* sV = sK + BN * LD;

    const int b = blockIdx.z, h = blockIdx.y;
    const int qb = gridDim.x - 1 - blockIdx.x;
    const SeqInfo si = seq_info(p, b);
    const int q0 = qb * BM;
    if (q0 >= si.lq) return;
    const int hk = h / (p.heads / p.kv_heads);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;

    const __nv_bfloat16* qg = p.q + b * p.qs[0] + h * p.qs[1] + static_cast<int64_t>(si.q_off) * p.qs[2];
    const __nv_bfloat16* dog = p.dout + b * p.dos[0] + h * p.dos[1] + static_cast<int64_t>(si.q_off) * p.dos[2];
    const __nv_bfloat16* kg = p.k + b * p.ks[0] + hk * p.ks[1] + static_cast<int64_t>(si.k_off) * p.ks[2];
    const __nv_bfloat16* vg = p.v + b * p.vs[0] + hk * p.vs[1] + static_cast<int64_t>(si.k_off) * p.vs[2];

    load_tile<BM, DP, kThreads>(sQ, qg, p.qs[2], q0, si.lq, p.d);
    load_tile<BM, DP, kThreads>(sdO, dog, p.dos[2], q0, si.lq, p.dv);

    const int row_a = q0 + warp * 16 + g, row_b = row_a + 8;
    // Row terms; rows past the end are padding and get harmless values.
    const float* lg = p.lse + b * p.ls[0] + h * p.ls[1];
    const float* dl = p.delta + b * p.delta_bs + h * p.delta_hs + si.q_off;
    float lse2[2], delta[2];
    lse2[0] = row_a < si.lq ? lg[(si.q_off + row_a) * p.ls[2]] * kLog2e : INFINITY;
    lse2[1] = row_b < si.lq ? lg[(si.q_off + row_b) * p.ls[2]] * kLog2e : INFINITY;
    delta[0] = row_a < si.lq ? dl[row_a] : 0.f;
    delta[1] = row_b < si.lq ? dl[row_b] : 0.f;
    // A row that saw no key has lse = -inf; +inf makes every P of it exactly 0.
    if (lse2[0] == -INFINITY) lse2[0] = INFINITY;
    if (lse2[1] == -INFINITY) lse2[1] = INFINITY;

    int kend = si.klen;
    if (p.causal) {
        const int qlast = min(q0 + BM, si.lq) - 1;
        kend = min(kend, qlast + si.shift + 1);
    }

    float dq[DP / 8][4];
#pragma unroll
    for (int n = 0; n < DP / 8; ++n) dq[n][0] = dq[n][1] = dq[n][2] = dq[n][3] = 0.f;

    for (int k0 = 0; k0 < kend; k0 += BN) {
        __syncthreads();
        load_tile<BN, DP, kThreads>(sK, kg, p.ks[2], k0, si.klen, p.d);
        load_tile<BN, DP, kThreads>(sV, vg, p.vs[2], k0, si.klen, p.dv);
        __syncthreads();

        float s[BN / 8][4], dp[BN / 8][4];
#pragma unroll
        for (int n = 0; n < BN / 8; ++n) {
            s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
            dp[n][0] = dp[n][1] = dp[n][2] = dp[n][3] = 0.f;
        }
#pragma unroll
        for (int kk = 0; kk < DP / 16; ++kk) {
            uint32_t a[4], ad[4];
            load_a_frag<LD>(a, sQ, warp * 16, kk * 16, lane);
            load_a_frag<LD>(ad, sdO, warp * 16, kk * 16, lane);
#pragma unroll
            for (int n = 0; n < BN / 8; ++n) {
                uint32_t b0, b1;
                load_b_frag<LD>(b0, b1, sK, n * 8, kk * 16, lane);
                mma_bf16(s[n], a, b0, b1);
                load_b_frag<LD>(b0, b1, sV, n * 8, kk * 16, lane);
                mma_bf16(dp[n], ad, b0, b1);
            }
        }
#pragma unroll
        for (int n = 0; n < BN / 8; ++n) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = (e < 2) ? row_a : row_b;
                const int j = k0 + n * 8 + t * 2 + (e & 1);
                const float x = logit2(p, si, b, h, i, j, s[n][e]);
                const float pv = fast_exp2(x - lse2[e >> 1]);
                s[n][e] = pv * (dp[n][e] - delta[e >> 1]);  // dS
            }
        }
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
            uint32_t a[4];
            a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int n2 = 0; n2 < DP / 16; ++n2) {
                uint32_t r[4];
                load_bt_frag<LD>(r, sK, kk * 16, n2 * 16, lane);
                mma_bf16(dq[2 * n2], a, r[0], r[1]);
                mma_bf16(dq[2 * n2 + 1], a, r[2], r[3]);
            }
        }
    }

    __syncthreads();
    __nv_bfloat16* so = sQ + warp * 16 * LD;
#pragma unroll
    for (int n = 0; n < DP / 8; ++n) {
        *reinterpret_cast<uint32_t*>(&so[g * LD + n * 8 + t * 2]) =
            pack_bf16(dq[n][0] * p.scale, dq[n][1] * p.scale);
        *reinterpret_cast<uint32_t*>(&so[(g + 8) * LD + n * 8 + t * 2]) =
            pack_bf16(dq[n][2] * p.scale, dq[n][3] * p.scale);
    }
    __syncwarp();
    __nv_bfloat16* dqg = p.dq + b * p.dqs[0] + h * p.dqs[1] + static_cast<int64_t>(si.q_off) * p.dqs[2];
    store_tile<16, DP, 32>(so, dqg, p.dqs[2], q0 + warp * 16, si.lq, p.d, lane);
}

// dK / dV: one CTA per (64 keys, kv head, batch); streams the query blocks of every
// query head in the group. WANT_DK / WANT_DV let a wide head dim run as two passes.
template <int DP, int BQ, bool WANT_DK, bool WANT_DV>
__global__ void __launch_bounds__(kThreads) bwd_dkv_kernel(const AttnParams p) {
    constexpr int BN = 64;
    constexpr int LD = DP + kPad;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* sV = sK + BN * LD;
    __nv_bfloat16* sQ = sV + BN * LD;
    __nv_bfloat16* sdO = sQ + BQ * LD;
    float* sLse = reinterpret_cast<float*>(sdO + BQ * LD);
    float* sDelta = sLse + BQ;

    const int b = blockIdx.z, hk = blockIdx.y;
    const SeqInfo si = seq_info(p, b);
    const int k0 = blockIdx.x * BN;
    if (k0 >= si.lk) return;
    const int group = p.heads / p.kv_heads;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;

    const __nv_bfloat16* kg = p.k + b * p.ks[0] + hk * p.ks[1] + static_cast<int64_t>(si.k_off) * p.ks[2];
    const __nv_bfloat16* vg = p.v + b * p.vs[0] + hk * p.vs[1] + static_cast<int64_t>(si.k_off) * p.vs[2];
    load_tile<BN, DP, kThreads>(sK, kg, p.ks[2], k0, si.klen, p.d);
    load_tile<BN, DP, kThreads>(sV, vg, p.vs[2], k0, si.klen, p.dv);

    const int key_a = k0 + warp * 16 + g, key_b = key_a + 8;

    float dk[WANT_DK ? DP / 8 : 1][4], dv[WANT_DV ? DP / 8 : 1][4];
#pragma unroll
    for (int n = 0; n < (WANT_DK ? DP / 8 : 1); ++n) dk[n][0] = dk[n][1] = dk[n][2] = dk[n][3] = 0.f;
#pragma unroll
    for (int n = 0; n < (WANT_DV ? DP / 8 : 1); ++n) dv[n][0] = dv[n][1] = dv[n][2] = dv[n][3] = 0.f;

    // First query row that can see key k0 (causal: j <= i + shift), rounded to a block.
    int qstart = 0;
    if (p.causal) {
        const int first = k0 - si.shift;
        qstart = first > 0 ? (first / BQ) * BQ : 0;
    }
    const bool any_key = k0 < si.klen;  // keys past the length get exact zeros

    for (int gi = 0; gi < group && any_key; ++gi) {
        const int h = hk * group + gi;
        const __nv_bfloat16* qg = p.q + b * p.qs[0] + h * p.qs[1] + static_cast<int64_t>(si.q_off) * p.qs[2];
        const __nv_bfloat16* dog = p.dout + b * p.dos[0] + h * p.dos[1] + static_cast<int64_t>(si.q_off) * p.dos[2];
        const float* lg = p.lse + b * p.ls[0] + h * p.ls[1];
        const float* dl = p.delta + b * p.delta_bs + h * p.delta_hs + si.q_off;

        for (int q0 = qstart; q0 < si.lq; q0 += BQ) {
            __syncthreads();
            load_tile<BQ, DP, kThreads>(sQ, qg, p.qs[2], q0, si.lq, p.d);
            load_tile<BQ, DP, kThreads>(sdO, dog, p.dos[2], q0, si.lq, p.dv);
            if (threadIdx.x < BQ) {
                const int i = q0 + threadIdx.x;
                float l2 = i < si.lq ? lg[(si.q_off + i) * p.ls[2]] * kLog2e : INFINITY;
                if (l2 == -INFINITY) l2 = INFINITY;  // a row without keys: P exactly 0
                sLse[threadIdx.x] = l2;
                sDelta[threadIdx.x] = i < si.lq ? dl[i] : 0.f;
            }
            __syncthreads();

            // S^T (keys x queries) and dP^T for this warp's 16 keys.
            float s[BQ / 8][4], dp[BQ / 8][4];
#pragma unroll
            for (int n = 0; n < BQ / 8; ++n) {
                s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
                dp[n][0] = dp[n][1] = dp[n][2] = dp[n][3] = 0.f;
            }
#pragma unroll
            for (int kk = 0; kk < DP / 16; ++kk) {
                uint32_t a[4], av[4];
                load_a_frag<LD>(a, sK, warp * 16, kk * 16, lane);
                load_a_frag<LD>(av, sV, warp * 16, kk * 16, lane);
#pragma unroll
                for (int n = 0; n < BQ / 8; ++n) {
                    uint32_t b0, b1;
                    load_b_frag<LD>(b0, b1, sQ, n * 8, kk * 16, lane);
                    mma_bf16(s[n], a, b0, b1);
                    load_b_frag<LD>(b0, b1, sdO, n * 8, kk * 16, lane);
                    mma_bf16(dp[n], av, b0, b1);
                }
            }
#pragma unroll
            for (int n = 0; n < BQ / 8; ++n) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = (e < 2) ? key_a : key_b;
                    const int il = n * 8 + t * 2 + (e & 1);
                    const int i = q0 + il;
                    float pv = 0.f;
                    if (i < si.lq) {
                        const float x = logit2(p, si, b, h, i, j, s[n][e]);
                        pv = fast_exp2(x - sLse[il]);
                    }
                    s[n][e] = pv;                               // P^T
                    dp[n][e] = pv * (dp[n][e] - sDelta[il]);    // dS^T
                }
            }
#pragma unroll
            for (int kk = 0; kk < BQ / 16; ++kk) {
                uint32_t ap[4], as[4];
                ap[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
                ap[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
                ap[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                ap[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
                as[0] = pack_bf16(dp[2 * kk][0], dp[2 * kk][1]);
                as[1] = pack_bf16(dp[2 * kk][2], dp[2 * kk][3]);
                as[2] = pack_bf16(dp[2 * kk + 1][0], dp[2 * kk + 1][1]);
                as[3] = pack_bf16(dp[2 * kk + 1][2], dp[2 * kk + 1][3]);
#pragma unroll
                for (int n2 = 0; n2 < DP / 16; ++n2) {
                    uint32_t r[4];
                    if constexpr (WANT_DV) {
                        load_bt_frag<LD>(r, sdO, kk * 16, n2 * 16, lane);
                        mma_bf16(dv[2 * n2], ap, r[0], r[1]);
                        mma_bf16(dv[2 * n2 + 1], ap, r[2], r[3]);
                    }
                    if constexpr (WANT_DK) {
                        load_bt_frag<LD>(r, sQ, kk * 16, n2 * 16, lane);
                        mma_bf16(dk[2 * n2], as, r[0], r[1]);
                        mma_bf16(dk[2 * n2 + 1], as, r[2], r[3]);
                    }
                }
            }
        }
    }

    // Stage through this warp's rows of sK / sV (no longer needed) and write out.
    __syncthreads();
    if constexpr (WANT_DV) {
        __nv_bfloat16* so = sV + warp * 16 * LD;
#pragma unroll
        for (int n = 0; n < DP / 8; ++n) {
            *reinterpret_cast<uint32_t*>(&so[g * LD + n * 8 + t * 2]) = pack_bf16(dv[n][0], dv[n][1]);
            *reinterpret_cast<uint32_t*>(&so[(g + 8) * LD + n * 8 + t * 2]) = pack_bf16(dv[n][2], dv[n][3]);
        }
        __syncwarp();
        __nv_bfloat16* dvg = p.dv_out + b * p.dvs[0] + hk * p.dvs[1] + static_cast<int64_t>(si.k_off) * p.dvs[2];
        store_tile<16, DP, 32>(so, dvg, p.dvs[2], k0 + warp * 16, si.lk, p.dv, lane);
    }
    if constexpr (WANT_DK) {
        __nv_bfloat16* so = sK + warp * 16 * LD;
#pragma unroll
        for (int n = 0; n < DP / 8; ++n) {
            *reinterpret_cast<uint32_t*>(&so[g * LD + n * 8 + t * 2]) =
                pack_bf16(dk[n][0] * p.scale, dk[n][1] * p.scale);
            *reinterpret_cast<uint32_t*>(&so[(g + 8) * LD + n * 8 + t * 2]) =
                pack_bf16(dk[n][2] * p.scale, dk[n][3] * p.scale);
        }
        __syncwarp();
        __nv_bfloat16* dkg = p.dk + b * p.dks[0] + hk * p.dks[1] + static_cast<int64_t>(si.k_off) * p.dks[2];
        store_tile<16, DP, 32>(so, dkg, p.dks[2], k0 + warp * 16, si.lk, p.d, lane);
    }
}


template <int DP, int BN>
int launch_dq(const AttnParams& p, cudaStream_t stream) {
    constexpr int smem = (2 * 64 + 2 * BN) * (DP + kPad) * 2;
    if (int rc = ensure_smem(bwd_dq_kernel<DP, BN>, smem, "cudaFuncSetAttribute(bwd_dq)")) return rc;
    dim3 grid((p.sq + 63) / 64, p.heads, p.batch);
    bwd_dq_kernel<DP, BN><<<grid, kThreads, smem, stream>>>(p);
    return check_cuda(cudaGetLastError(), "bwd_dq launch");
}

template <int DP, int BQ, bool DK, bool DV>
int launch_dkv(const AttnParams& p, cudaStream_t stream) {
    constexpr int smem = (2 * 64 + 2 * BQ) * (DP + kPad) * 2 + 2 * BQ * 4;
    if (int rc = ensure_smem(bwd_dkv_kernel<DP, BQ, DK, DV>, smem, "cudaFuncSetAttribute(bwd_dkv)")) return rc;
    dim3 grid((p.sk + 63) / 64, p.kv_heads, p.batch);
    bwd_dkv_kernel<DP, BQ, DK, DV><<<grid, kThreads, smem, stream>>>(p);
    return check_cuda(cudaGetLastError(), "bwd_dkv launch");
}

}  // namespace

int launch_backward_delta(const AttnParams& p, cudaStream_t stream) {
    const int64_t ncounters = p.dkv_counters ? backward_counter_count(p, p.gsplit) : 0;
    const bool aligned =
        ((reinterpret_cast<uintptr_t>(p.out) | reinterpret_cast<uintptr_t>(p.dout)) & 15) == 0 &&
        ((p.os[0] | p.os[1] | p.os[2] | p.dos[0] | p.dos[1] | p.dos[2]) & 7) == 0;
    if (aligned && (p.dv == 64 || p.dv == 128)) {
        const int rows = p.dv == 64 ? 32 : 16;
        dim3 grid((p.sq + rows - 1) / rows, p.heads, p.batch);
        if (p.dv == 64) {
            bwd_delta_vec_kernel<64><<<grid, 256, 0, stream>>>(p, ncounters);
        } else {
            bwd_delta_vec_kernel<128><<<grid, 256, 0, stream>>>(p, ncounters);
        }
        return check_cuda(cudaGetLastError(), "bwd_delta launch");
    }
    dim3 grid((p.sq + 3) / 4, p.heads, p.batch);
    bwd_delta_kernel<<<grid, kThreads, 0, stream>>>(p, ncounters);
    return check_cuda(cudaGetLastError(), "bwd_delta launch");
}

int launch_backward_mma(const AttnParams& p, cudaStream_t stream) {
    if (int rc = launch_backward_delta(p, stream)) return rc;
    const int dmax = p.d > p.dv ? p.d : p.dv;
    int rc;
    if (dmax <= 32) {
        if ((rc = launch_dq<32, 64>(p, stream))) return rc;
        return launch_dkv<32, 64, true, true>(p, stream);
    }
    if (dmax <= 64) {
        if ((rc = launch_dq<64, 64>(p, stream))) return rc;
        return launch_dkv<64, 64, true, true>(p, stream);
    }
    if (dmax <= 128) {
        if ((rc = launch_dq<128, 32>(p, stream))) return rc;
        return launch_dkv<128, 32, true, true>(p, stream);
    }
    if (dmax <= 256) {
        if ((rc = launch_dq<256, 32>(p, stream))) return rc;
        if ((rc = launch_dkv<256, 32, true, false>(p, stream))) return rc;
        return launch_dkv<256, 32, false, true>(p, stream);
    }
    return fail(KTT_B200_ERR_UNSUPPORTED, "head dim %d exceeds 256", dmax);
}

}  // namespace ktt
