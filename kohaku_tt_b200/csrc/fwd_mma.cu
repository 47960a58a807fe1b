// General forward kernel on warp-level MMA (mma.sync m16n8k16 bf16 -> fp32).
//
// Covers everything the operator surface accepts: any head dim up to 256 (zero-padded in
// shared memory), MHA / GQA / MQA, arbitrary batch / head / row strides, additive and
// boolean masks with broadcast strides, per-batch key lengths, top-left and bottom-right
// causal, packed sequences by cu_seqlens. It is the kernel behind every shape the
// TMA + tcgen05 kernel does not take, and the yardstick that kernel is compared with.
//
// Algorithm (the single-pass flash forward of ktt_flash/compute.cpp:193-491 restated for
// a CUDA warp): per 64-row query block, stream key/value blocks; S = Q K^T in fp32;
// base-2 online softmax with fp32 running max and sum; P rounded to bf16; O += P V in
// fp32; O / l and lse = ln2 * (m + log2 l) at the end.
#include "tiles.cuh"

namespace ktt {
namespace {

constexpr int kBM = 64;       // query rows per CTA (16 per warp)
constexpr int kThreads = 128;

template <int DP, int BN>
__global__ void __launch_bounds__(kThreads, DP <= 64 ? 4 : 1) fwd_mma_kernel(const AttnParams p) {
    constexpr int LD = DP + kPad;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* sK = sQ + kBM * LD;
    __nv_bfloat16* sV = sK + BN * LD;

    const int b = blockIdx.z, h = blockIdx.y;
    const int qb = gridDim.x - 1 - blockIdx.x;  // longest causal rows first
    const SeqInfo si = seq_info(p, b);
    const int q0 = qb * kBM;
    if (q0 >= si.lq) return;
    const int hk = h / (p.heads / p.kv_heads);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;

    const __nv_bfloat16* qg = p.q + b * p.qs[0] + h * p.qs[1] + static_cast<int64_t>(si.q_off) * p.qs[2];
    const __nv_bfloat16* kg = p.k + b * p.ks[0] + hk * p.ks[1] + static_cast<int64_t>(si.k_off) * p.ks[2];
    const __nv_bfloat16* vg = p.v + b * p.vs[0] + hk * p.vs[1] + static_cast<int64_t>(si.k_off) * p.vs[2];

    load_tile<kBM, DP, kThreads>(sQ, qg, p.qs[2], q0, si.lq, p.d);

    // Keys this block can see at all.
    int kend = si.klen;
    if (p.causal) {
        const int qlast = min(q0 + kBM, si.lq) - 1;
        kend = min(kend, qlast + si.shift + 1);
    }

    float o[DP / 8][4];
#pragma unroll
    for (int n = 0; n < DP / 8; ++n) {
        o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    }
    float m_run[2] = {-INFINITY, -INFINITY};
    float l_run[2] = {0.f, 0.f};
    const int row_a = q0 + warp * 16 + g;  // this thread's two query rows
    const int row_b = row_a + 8;

    for (int k0 = 0; k0 < kend; k0 += BN) {
        __syncthreads();  // previous tile fully consumed (and sQ written on the first pass)
        load_tile<BN, DP, kThreads>(sK, kg, p.ks[2], k0, si.klen, p.d);
        load_tile<BN, DP, kThreads>(sV, vg, p.vs[2], k0, si.klen, p.dv);
        __syncthreads();

        float s[BN / 8][4];
#pragma unroll
        for (int n = 0; n < BN / 8; ++n) {
            s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
        }
        // The tile's mask terms, requested before the score MMAs so that they arrive
        // meanwhile.
        float mk[BN / 8][4];
        const bool has_mask = p.mask_dtype != KTT_B200_MASK_NONE;
#pragma unroll
        for (int n = 0; n < BN / 8; ++n) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                mk[n][e] = has_mask ? mask_term(p, si, b, h, (e < 2) ? row_a : row_b, k0 + n * 8 + t * 2 + (e & 1)) : 0.f;
            }
        }
#pragma unroll
        for (int kk = 0; kk < DP / 16; ++kk) {
            uint32_t a[4];
            load_a_frag<LD>(a, sQ, warp * 16, kk * 16, lane);
#pragma unroll
            for (int n = 0; n < BN / 8; ++n) {
                uint32_t b0, b1;
                load_b_frag<LD>(b0, b1, sK, n * 8, kk * 16, lane);
                mma_bf16(s[n], a, b0, b1);
            }
        }

        // Logits and the tile's row maxima.
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < BN / 8; ++n) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = (e < 2) ? row_a : row_b;
                const int j = k0 + n * 8 + t * 2 + (e & 1);
                const float x = logit2_with(p, si, i, j, s[n][e], mk[n][e]);
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
            alpha[r] = fast_exp2(m_run[r] - m_use[r]);  // exp2(-inf) = 0 on the first tile
            m_run[r] = m_new;
            l_run[r] *= alpha[r];
        }
#pragma unroll
        for (int n = 0; n < DP / 8; ++n) {
            o[n][0] *= alpha[0];
            o[n][1] *= alpha[0];
            o[n][2] *= alpha[1];
            o[n][3] *= alpha[1];
        }
#pragma unroll
        for (int n = 0; n < BN / 8; ++n) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float pv = fast_exp2(s[n][e] - m_use[e >> 1]);
                s[n][e] = pv;
                l_run[e >> 1] += pv;
            }
        }
        // O += P V with P as bf16 A-fragments taken straight from the accumulators.
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
                load_bt_frag<LD>(r, sV, kk * 16, n2 * 16, lane);
                mma_bf16(o[2 * n2], a, r[0], r[1]);
                mma_bf16(o[2 * n2 + 1], a, r[2], r[3]);
            }
        }
    }

    // Finalize: full row sums, normalize, statistics.
    float inv[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
        inv[r] = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
    }
    if (p.lse && t == 0) {
        float* lg = p.lse + b * p.ls[0] + h * p.ls[1];
        if (row_a < si.lq) {
            lg[(si.q_off + row_a) * p.ls[2]] =
                l_run[0] > 0.f ? kLn2 * (m_run[0] + log2f(l_run[0])) : -INFINITY;
        }
        if (row_b < si.lq) {
            lg[(si.q_off + row_b) * p.ls[2]] =
                l_run[1] > 0.f ? kLn2 * (m_run[1] + log2f(l_run[1])) : -INFINITY;
        }
    }
    // Stage this warp's 16 output rows in its own rows of sQ, then write them out.
    __syncthreads();  // every warp is done reading sQ as the A operand
    __nv_bfloat16* so = sQ + warp * 16 * LD;
#pragma unroll
    for (int n = 0; n < DP / 8; ++n) {
        *reinterpret_cast<uint32_t*>(&so[g * LD + n * 8 + t * 2]) =
            pack_bf16(o[n][0] * inv[0], o[n][1] * inv[0]);
        *reinterpret_cast<uint32_t*>(&so[(g + 8) * LD + n * 8 + t * 2]) =
            pack_bf16(o[n][2] * inv[1], o[n][3] * inv[1]);
    }
    __syncwarp();
    __nv_bfloat16* og = p.out + b * p.os[0] + h * p.os[1] + static_cast<int64_t>(si.q_off) * p.os[2];
    store_tile<16, DP, 32>(so, og, p.os[2], q0 + warp * 16, si.lq, p.dv, lane);
}

template <int DP, int BN>
int launch(const AttnParams& p, cudaStream_t stream) {
    constexpr int smem = (kBM + 2 * BN) * (DP + kPad) * 2;
    if (int rc = ensure_smem(fwd_mma_kernel<DP, BN>, smem, "cudaFuncSetAttribute(fwd_mma)")) return rc;
    dim3 grid((p.sq + kBM - 1) / kBM, p.heads, p.batch);
    fwd_mma_kernel<DP, BN><<<grid, kThreads, smem, stream>>>(p);
    return check_cuda(cudaGetLastError(), "fwd_mma launch");
}

}  // namespace

int launch_forward_mma(const AttnParams& p, cudaStream_t stream) {
    const int dmax = p.d > p.dv ? p.d : p.dv;
    if (dmax <= 32) return launch<32, 64>(p, stream);
    if (dmax <= 64) return launch<64, 64>(p, stream);
    if (dmax <= 128) return launch<128, 64>(p, stream);
    if (dmax <= 256) return launch<256, 32>(p, stream);
    return fail(KTT_B200_ERR_UNSUPPORTED, "head dim %d exceeds 256", dmax);
}

}  // namespace ktt
