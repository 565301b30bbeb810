// Backward kernels, bf16, sm_100a.  The [T, E*d_e] intermediate is recomputed block by block.
//
//   M = Q K^T, N = Q U^T, sg = sigmoid(M), s = M*sg, dA = dO V^T          (per 64-row weight block)
//   dR_e = rowsum(dA*s*N), dM = dA*(r*N)*(sg + s*(1-sg)), dN = dA*s*r, A = s*N*r
//   dQ += dM K + dN U ;  dK = sum_t dM^T Q ;  dU = sum_t dN^T Q ;  dV = sum_t A^T dO
//
// Two kernels, each the sole owner of its accumulators (no floating-point atomics, bit-reproducible):
//
// bwd_dq_kernel  -- token-stationary.  One CTA owns 128 token rows of one (batch, head): its Q and dO
//   tiles are copied once into tensor memory and all three MMA chains read their A operand from there,
//   the head's weights stream through shared memory (K/U ring of 3, V ring of 2).
//   Tensor memory: dQ accumulator (128 cols), Q and dO as bf16 (64 + 64), S = [M|N] (128), dA (64), and the
//   bf16 [dM|dN] operand of the dQ update (64).  Produces dQ (TMA store) and dR (direct stores).
//
// bwd_dw_kernel  -- weight-stationary.  One CTA owns one 64-row block of K, U and V of one K/U/V
//   head and a contiguous range of token tiles (the token axis is split `nsplit` ways to fill the
//   machine).  Weights stay in shared memory, {Q, dO} tiles stream through a ring of 2.
//   Tensor memory: [dK;dU] accumulator (128 lanes), dV accumulator (transposed, d_h x 64, when d_h = 128; else
//   M = 64), two S buffers and one dA buffer (the element-wise warps copy dA to registers first and hand it
//   back at once), so that the recompute of tile i+1 runs under the element-wise math of tile i.
//   Each CTA writes fp32 partial sums to the workspace; dw_reduce_kernel adds the splits in a fixed
//   order and writes bf16 dK, dU, dV.
//
// Both use 384 threads: warp 0 TMA producer, warps 1 and 3 MMA issuers (one per MMA chain; warp 1 owns
// tensor memory), warps 4-11 element-wise math (warp % 4 = TMEM lane quarter, (warp-4)/4 = which 32 of the 64 block columns).
#include <atomic>
#include <mutex>
#include <queue>
#include <vector>

#include "kernels.h"
#include "tc_common.cuh"
#include "tensormap.cuh"

namespace fmhf {
namespace {

#ifndef FMHF_BWD_PARTS
#define FMHF_BWD_PARTS 2
#endif
// Element-wise warps: 4 lane quarters x kParts column parts of a 64-column block (a thread = one token row x
// kCols columns).  More, narrower threads shorten the arithmetic phase of a block; the fixed part of a block's
// element-wise step (barrier waits, tensor-memory load and store latencies) does not shrink.
constexpr int kParts = FMHF_BWD_PARTS, kCols = 64 / kParts, kSubs = kCols / 16;
constexpr int kBT = 128, kBI = 64, kActThreads = 128 * kParts, kThreads = 128 + kActThreads;
constexpr int kEpiThreads = 256;  // the warps of column parts 0 and 1 write the accumulators out
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTile = kBT * 128;    // one 128-row x 64-col SW128 chunk: 16 KB
constexpr uint32_t kWChunk = kBI * 128;  // one 64-row x 64-col chunk: 8 KB

// Element-wise backward math for two neighbouring intermediate columns of one token row, on packed
// fp32 pairs.  m, n are the raw products Q K^T, Q U^T; with the layer's constants s0 (head), s1 (up),
// s2 (final) the forward is A = silu(s0 m) (s1 n) s2 r.  With t = tanh(s0 m / 2): sg = sigmoid(s0 m) =
// 0.5 + 0.5 t, s = m*sg (so silu(s0 m) = s0 s), silu'(s0 m) = sg + s * s0 (1 - sg).  All three constants
// fold into the per-row factor r2 = s0 s1 s2 r and into the two constants below, at no cost per element:
//   dM = dA r2 n silu'(s0 m),  dN = dA r2 s,  A = s n r2,  dR = s0 s1 s2 * sum dA s n.
struct BwdConst {
    f32x2 half_s0, p_half_s0, n_half_s0;  // (s0/2), (s0/2), (-s0/2): tanh argument scale and s0 (1 - sg) = s0/2 - (s0/2) t
};
__device__ __forceinline__ BwdConst bwd_const(float s0) {
    return BwdConst{f2_pack(0.5f * s0, 0.5f * s0), f2_pack(0.5f * s0, 0.5f * s0), f2_pack(-0.5f * s0, -0.5f * s0)};
}
struct BwdPair {
    f32x2 dm, dn, sn, da;  // dM, dN, s*N (times r2 gives A, times dA sums to dR / (s0 s1 s2)), dA
};
__device__ __forceinline__ BwdPair bwd_pair(f32x2 m, f32x2 n, f32x2 da, f32x2 r2, const BwdConst &k) {
    const f32x2 half = f2_pack(0.5f, 0.5f);
    const f32x2 t = f2_tanh(f2_mul(m, k.half_s0));
    const f32x2 sg = f2_fma(t, half, half);
    const f32x2 omsg = f2_fma(t, k.n_half_s0, k.p_half_s0);
    const f32x2 s = f2_mul(m, sg);
    const f32x2 dsilu = f2_fma(s, omsg, sg);
    const f32x2 dar = f2_mul(da, r2);
    BwdPair o;
    o.sn = f2_mul(s, n);
    o.dn = f2_mul(dar, s);
    o.dm = f2_mul(f2_mul(dar, n), dsilu);
    o.da = da;
    return o;
}

// =============================================================================================
//                                       dQ / dR kernel
// =============================================================================================
template <int DH>
struct DqSmem {
    static constexpr int kChunks = (DH + 63) / 64;
    static constexpr uint32_t kQBytes = kChunks * kTile;
    static constexpr uint32_t kKUStage = kChunks * 2 * kWChunk;  // per chunk: [K;U] = 128 rows
    static constexpr uint32_t kVStage = kChunks * kWChunk;
    static constexpr int kKUStages = 3, kVStages = 2;
    static constexpr uint32_t kOffQ = 0;
    static constexpr uint32_t kOffdO = kOffQ + kQBytes;
    static constexpr uint32_t kOffKU = kOffdO + kQBytes;
    static constexpr uint32_t kOffV = kOffKU + kKUStages * kKUStage;
    static constexpr uint32_t kOffCtl = kOffV + kVStages * kVStage;
    static constexpr uint32_t kCtlBytes = 256 + 2 * (kParts - 1) * 128 * 4;  // barriers + two sets of dR exchange rows
    static constexpr uint32_t kTotal = kOffCtl + kCtlBytes + 1024;
};

// Barriers.  Q and dO are copied once into tensor memory (QT); S, dA and the [dM|dN] operand each have ONE buffer
// there, because the accumulator, Q and dO take half of tensor memory:
//   SFULL (S and dA of the block computed: one commit from each of their issuers), SEMPTY (both are in the
//   element-wise warps' registers), PFULL ([dM|dN] written), PEMPTY (the dQ update that read it is done).
// All of them complete once per block and every waiter waits on every phase, so a one-bit parity is enough.
enum { DQ_QFULL = 0, DQ_KUFULL = 1, DQ_KUEMPTY = 4, DQ_VFULL = 7, DQ_VEMPTY = 9, DQ_SFULL = 11, DQ_SEMPTY = 12,
       DQ_PFULL = 13, DQ_PEMPTY = 14, DQ_ACCFULL = 15, DQ_QT = 16, DQ_DRFULL = 18, DQ_DRFREE = 20, DQ_BARS = 22 };

struct DqArgs {
    const float *R;
    long long r_sb, r_sh, r_ss;
    float *dR;
    long long dr_sb, dr_sh, dr_ss;
    int S, E, De, G;
    float s0, c;  // head_scaling; head_scaling * up_scaling * final_scaling
    WaitArgs wait;
};

template <int DH>
__global__ void __launch_bounds__(kThreads, 1)
bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
              const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmU,
              const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdQ, const DqArgs args) {
    using L = DqSmem<DH>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *gbase = smem_raw + (base - raw);
    const uint32_t sQ = base + L::kOffQ, sdO = base + L::kOffdO, sKU = base + L::kOffKU, sV = base + L::kOffV,
                   sBar = base + L::kOffCtl;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(gbase + L::kOffCtl + DQ_BARS * 8);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(gbase + L::kOffCtl + DQ_BARS * 8 + 4);
    volatile float *drx = reinterpret_cast<volatile float *>(gbase + L::kOffCtl + 256);  // [2][kParts - 1][128]
    auto bar = [&](int i) { return sBar + 8u * i; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = blockIdx.x * kBT, h = blockIdx.y, b = blockIdx.z, hk = h / args.G;
    const int bpe = args.De / kBI, nblk = args.E * bpe;
    const WaitCtl ctl{abort_flag, args.wait};
    constexpr int W = kKernelBwdDq * 100;
    // Tensor memory: dQ accumulator, Q and dO as bf16 A operands (64 columns each), S = [M | N], dA, [dM | dN] (bf16).
    constexpr uint32_t kColAcc = 0, kColQ = 128, kColdO = 192, kColS = 256, kColdA = 384, kColP = 448;

    if (threadIdx.x == 0) {
        *abort_flag = launch_aborted(args.wait);  // a CTA of this launch gave up: drain fast
        mbar_init(bar(DQ_QFULL), 1);
        for (int s = 0; s < L::kKUStages; ++s) { mbar_init(bar(DQ_KUFULL + s), 1); mbar_init(bar(DQ_KUEMPTY + s), 1); }
        for (int s = 0; s < L::kVStages; ++s) { mbar_init(bar(DQ_VFULL + s), 1); mbar_init(bar(DQ_VEMPTY + s), 1); }
        mbar_init(bar(DQ_SFULL), 2);                          // one commit from each of the two recompute issuers
        mbar_init(bar(DQ_SEMPTY), arrivals_of(kActThreads));  // S and dA are in registers
        mbar_init(bar(DQ_PFULL), arrivals_of(kActThreads));   // [dM|dN] written
        mbar_init(bar(DQ_PEMPTY), 1);                         // the dQ update that read [dM|dN] is done
        mbar_init(bar(DQ_QT), arrivals_of(kActThreads));      // Q and dO copied to tensor memory
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar(DQ_DRFULL + i), arrivals_of(kActThreads - 128));  // column parts 1.. have written their dR_e partials
            mbar_init(bar(DQ_DRFREE + i), arrivals_of(128));                 // part 0 has read them: the rows may be reused
        }
        mbar_init(bar(DQ_ACCFULL), 1);
        fence_mbar_init();
    }
    if (warp == 1) tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const bool dead = *abort_flag != 0;

    if (dead) {
        // nothing: fall through to the teardown
    } else if (warp == 0) {
        if (lane == 0) {
            tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmdO); tma_prefetch_desc(&tmK);
            tma_prefetch_desc(&tmU); tma_prefetch_desc(&tmV);
            mbar_arrive_expect_tx(bar(DQ_QFULL), 2 * L::kQBytes);
            for (int c = 0; c < L::kChunks; ++c) {
                tma_load_4d(sQ + c * kTile, &tmQ, bar(DQ_QFULL), c * 64, t0, h, b);
                tma_load_4d(sdO + c * kTile, &tmdO, bar(DQ_QFULL), c * 64, t0, h, b);
            }
            int sk = 0, sv = 0;
            uint32_t phk = 1, phv = 1;
            for (int j = 0; j < nblk; ++j) {
                const int row = j * kBI;
                if (!mbar_wait(bar(DQ_KUEMPTY + sk), phk, ctl, W + 1)) break;
                const uint32_t fk = bar(DQ_KUFULL + sk);
                mbar_arrive_expect_tx(fk, L::kKUStage);
#pragma unroll
                for (int c = 0; c < L::kChunks; ++c) {
                    const uint32_t d = sKU + sk * L::kKUStage + c * 2 * kWChunk;
                    tma_load_3d(d, &tmK, fk, c * 64, row, hk);
                    tma_load_3d(d + kWChunk, &tmU, fk, c * 64, row, hk);
                }
                if (!mbar_wait(bar(DQ_VEMPTY + sv), phv, ctl, W + 2)) break;
                const uint32_t fv = bar(DQ_VFULL + sv);
                mbar_arrive_expect_tx(fv, L::kVStage);
#pragma unroll
                for (int c = 0; c < L::kChunks; ++c)
                    tma_load_3d(sV + sv * L::kVStage + c * kWChunk, &tmV, fv, c * 64, row, hk);
                if (++sk == L::kKUStages) { sk = 0; phk ^= 1; }
                if (++sv == L::kVStages) { sv = 0; phv ^= 1; }
            }
        }
    } else if (warp == 1) {
        // Three MMA chains, three issuing threads (warps 1, 2, 3), so that none waits on another's barriers and the
        // tensor pipe, which accepts MMAs only a few ahead of execution, is fed by whichever is ready.  Every chain
        // reads its A operand from tensor memory: an MMA with both operands in shared memory takes the SM's whole
        // shared-memory bandwidth (8 KB per 64 clk), which the weight tiles arriving by TMA need as well.
        // Issuer 1: S = Q [K;U]^T.
        if (lane == 0) {
            constexpr uint32_t idS = umma_idesc(128, 2 * kBI, false, false);
            const uint64_t dKU0 = desc_kmajor(sKU);
            constexpr uint64_t kKUStep = L::kKUStage >> 4;
            bool ok = mbar_wait(bar(DQ_QT), 0, ctl, W + 3);
            int sk = 0;
            uint32_t phk = 0;
            for (int j = 0; ok && j < nblk; ++j) {
                if (!mbar_wait(bar(DQ_KUFULL + sk), phk, ctl, W + 4)) break;
                if (j >= 1 && !mbar_wait(bar(DQ_SEMPTY), (j - 1) & 1, ctl, W + 5)) break;
                tc_fence_after();
                const uint64_t dku = dKU0 + sk * kKUStep;
#pragma unroll
                for (int k = 0; k < DH / 16; ++k) {
                    const int c = k >> 2, kk = k & 3;
                    umma_ts(tmem + kColS, tmem + kColQ + k * 8, dku + ((c * 2 * kWChunk + kk * 32) >> 4), idS, k > 0 ? 1u : 0u);
                }
                umma_commit(bar(DQ_SFULL));
                if (++sk == L::kKUStages) { sk = 0; phk ^= 1; }
            }
        }
    } else if (warp == 2) {
        // Issuer 2: dA = dO V^T.
        if (lane == 0) {
            constexpr uint32_t idA = umma_idesc(128, kBI, false, false);
            const uint64_t dV0 = desc_kmajor(sV);
            constexpr uint64_t kVStep = L::kVStage >> 4;
            bool ok = mbar_wait(bar(DQ_QT), 0, ctl, W + 3);
            int sv = 0;
            uint32_t phv = 0;
            for (int j = 0; ok && j < nblk; ++j) {
                if (!mbar_wait(bar(DQ_VFULL + sv), phv, ctl, W + 4)) break;
                if (j >= 1 && !mbar_wait(bar(DQ_SEMPTY), (j - 1) & 1, ctl, W + 5)) break;
                tc_fence_after();
                const uint64_t dv = dV0 + sv * kVStep;
#pragma unroll
                for (int k = 0; k < DH / 16; ++k) {
                    const int c = k >> 2, kk = k & 3;
                    umma_ts(tmem + kColdA, tmem + kColdO + k * 8, dv + ((c * kWChunk + kk * 32) >> 4), idA, k > 0 ? 1u : 0u);
                }
                umma_commit(bar(DQ_VEMPTY + sv));
                umma_commit(bar(DQ_SFULL));
                if (++sv == L::kVStages) { sv = 0; phv ^= 1; }
            }
        }
    } else if (warp == 3) {
        // Issuer 3: dQ += [dM|dN] [K;U], with [dM|dN] read from tensor memory.
        if (lane == 0) {
            constexpr uint32_t idQ = umma_idesc(128, DH, false, true);
            const uint64_t dKUmn0 = desc_mnmajor(sKU, 2 * kWChunk);
            constexpr uint64_t kKUStep = L::kKUStage >> 4;
            int sk = 0;
            bool ok = true;
            for (int j = 0; j < nblk; ++j) {
                if (!mbar_wait(bar(DQ_PFULL), j & 1, ctl, W + 6)) { ok = false; break; }
                tc_fence_after();
                const uint64_t dku = dKUmn0 + sk * kKUStep;
                // [dM|dN] as packed bf16 pairs in 64 columns.  The thread that handled block columns [c, c + kCols) wrote
                // its dM to columns [c, c + kCols/2) and its dN to [c + kCols/2, c + kCols).  K step k (16 values = 8
                // columns; steps 0-3 pair with the K rows of the stage, 4-7 with the U rows) covers block columns
                // [16 (k%4), 16 (k%4) + 16).
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const int bc = 16 * (k & 3);
                    const int col = (bc / kCols) * kCols + (bc % kCols) / 2 + (k >> 2) * (kCols / 2);
                    umma_ts(tmem + kColAcc, tmem + kColP + col, dku + k * 128, idQ, (j > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(bar(DQ_KUEMPTY + sk));
                umma_commit(bar(DQ_PEMPTY));
                if (++sk == L::kKUStages) sk = 0;
            }
            if (ok) umma_commit(bar(DQ_ACCFULL));
        }
    } else if (warp >= 4) {
        const int quarter = warp & 3, part = (warp - 4) >> 2, half = part;  // part: which kCols of the block's 64 columns
        const int row = quarter * 32 + lane, t = t0 + row;
        const bool in_range = t < args.S;
        const float *rrow = args.R + (long long)b * args.r_sb + (long long)h * args.r_sh + (long long)t * args.r_ss;
        float *drrow = args.dR + (long long)b * args.dr_sb + (long long)h * args.dr_sh + (long long)t * args.dr_ss;
        const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
        bool ok = true;
        // Q and dO: shared -> tensor memory, once (thread = token row; column part p < 2 copies columns [64p, 64p + 64)
        // of d_h of both tiles).
        if (!mbar_wait(bar(DQ_QFULL), 0, ctl, W + 12)) ok = false;
        if (ok && part < 2 && part * 64 < DH) {
#pragma unroll
            for (int which = 0; which < 2; ++which) {
                uint32_t v32[32];
                const uint8_t *src = gbase + (which ? L::kOffdO : L::kOffQ) + part * kTile;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint4 v = *reinterpret_cast<const uint4 *>(src + sw128_offset(row, c));
                    v32[4 * c] = v.x; v32[4 * c + 1] = v.y; v32[4 * c + 2] = v.z; v32[4 * c + 3] = v.w;
                }
                tmem_st32(lane_base + (which ? kColdO : kColQ) + part * 32, v32);
            }
            tmem_st_wait();
        }
        tc_fence_before();
        warp_arrive(bar(DQ_QT));
        float r_cur = 0.f, r_next = in_range ? __ldg(rrow) : 0.f;
        f32x2 dr2 = f2_pack(0.f, 0.f);  // running dR_e of this thread's columns (two interleaved partial sums)
        const BwdConst kc = bwd_const(args.s0);
        int in_e = 0, e = 0;  // block index inside the current sub-network; current sub-network
        for (int j = 0; ok && j < nblk; ++j) {
            if (in_e == 0) {
                r_cur = r_next;
                r_next = (in_range && e + 1 < args.E) ? __ldg(rrow + e + 1) : 0.f;
                dr2 = f2_pack(0.f, 0.f);
            }
            if (!mbar_wait(bar(DQ_SFULL), j & 1, ctl, W + 7)) { ok = false; break; }
            tc_fence_after();
            const uint32_t tS = lane_base + kColS + part * kCols, tA = lane_base + kColdA + part * kCols;
            uint32_t pm[kCols / 2], pn[kCols / 2];  // packed bf16 pairs of dM, dN for this thread's columns
            const f32x2 r2 = f2_pack(args.c * r_cur, args.c * r_cur);
            if (kCols == 32) {
                // the whole part at once, so that S and dA are free for the next block before any arithmetic
                uint32_t m[32], n[32], da[32];
                tmem_ld32x3_sync(tS, tS + kBI, tA, m, n, da);
                tc_fence_before();
                warp_arrive(bar(DQ_SEMPTY));
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const BwdPair x = bwd_pair(f2_pack_bits(m[2 * i], m[2 * i + 1]), f2_pack_bits(n[2 * i], n[2 * i + 1]),
                                               f2_pack_bits(da[2 * i], da[2 * i + 1]), r2, kc);
                    dr2 = f2_fma(x.da, x.sn, dr2);
                    pm[i] = f2_to_bf16x2(x.dm);
                    pn[i] = f2_to_bf16x2(x.dn);
                }
            } else {
                uint32_t m[16], n[16], da[16];
                tmem_ld16x3_sync(tS, tS + kBI, tA, m, n, da);
                tc_fence_before();
                warp_arrive(bar(DQ_SEMPTY));
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const BwdPair x = bwd_pair(f2_pack_bits(m[2 * i], m[2 * i + 1]), f2_pack_bits(n[2 * i], n[2 * i + 1]),
                                               f2_pack_bits(da[2 * i], da[2 * i + 1]), r2, kc);
                    dr2 = f2_fma(x.da, x.sn, dr2);
                    pm[i] = f2_to_bf16x2(x.dm);
                    pn[i] = f2_to_bf16x2(x.dn);
                }
            }
            // the dQ update of the previous block has read the [dM|dN] buffer
            if (j >= 1 && !mbar_wait(bar(DQ_PEMPTY), (j - 1) & 1, ctl, W + 8)) { ok = false; break; }
            tc_fence_after();
            const uint32_t tP = lane_base + kColP + part * kCols;
            if (kCols == 32) {
                tmem_st16(tP, pm);
                tmem_st16(tP + 16, pn);
            } else {
                tmem_st8(tP, pm);
                tmem_st8(tP + 8, pn);
            }
            tmem_st_wait();
            tc_fence_before();
            warp_arrive(bar(DQ_PFULL));
            if (++in_e == bpe) {  // sub-network finished: add the column parts of dR_e, in part order
                const int xb = e & 1;
                float dr_lo, dr_hi;
                f2_unpack(dr2, dr_lo, dr_hi);
                const float dr_acc = (dr_lo + dr_hi) * args.c;
                volatile float *xrow = drx + (xb * (kParts - 1)) * 128 + row;
                if (part != 0) {
                    // the exchange rows of sub-network e were last used by e - 2: wait until those values have been read
                    if (e >= 2 && !mbar_wait(bar(DQ_DRFREE + xb), ((e >> 1) - 1) & 1, ctl, W + 11)) { ok = false; break; }
                    xrow[(part - 1) * 128] = dr_acc;
                    warp_arrive(bar(DQ_DRFULL + xb));
                } else {
                    if (!mbar_wait(bar(DQ_DRFULL + xb), (e >> 1) & 1, ctl, W + 9)) { ok = false; break; }
                    float sum = dr_acc;
#pragma unroll
                    for (int q = 0; q < kParts - 1; ++q) sum += xrow[q * 128];
                    warp_arrive(bar(DQ_DRFREE + xb));
                    if (in_range) drrow[e] = sum;
                }
                in_e = 0;
                ++e;
            }
        }
        if (part >= 2) ok = false;  // the accumulator is written out by the warps of parts 0 and 1
        if (ok) ok = mbar_wait(bar(DQ_ACCFULL), 0, ctl, W + 10);
        if (ok) {
            tc_fence_after();
            constexpr int kColsPerHalf = DH / 2;
            const int c0 = half * kColsPerHalf;
#pragma unroll
            for (int g = 0; g < kColsPerHalf / 16; ++g) {
                uint32_t o[16];
                tmem_ld16_sync(lane_base + kColAcc + c0 + g * 16, o);
#pragma unroll
                for (int v = 0; v < 2; ++v) {
                    const int col = c0 + g * 16 + v * 8;
                    const uint32_t dst = sQ + (col >> 6) * kTile + sw128_offset(row, (col & 63) >> 3);
                    st_shared_v4(dst, pack_bf16(__uint_as_float(o[8 * v + 0]), __uint_as_float(o[8 * v + 1])),
                                 pack_bf16(__uint_as_float(o[8 * v + 2]), __uint_as_float(o[8 * v + 3])),
                                 pack_bf16(__uint_as_float(o[8 * v + 4]), __uint_as_float(o[8 * v + 5])),
                                 pack_bf16(__uint_as_float(o[8 * v + 6]), __uint_as_float(o[8 * v + 7])));
                }
            }
            tc_fence_before();
            fence_async_smem();
        }
        if (part < 2) named_bar_sync(1, kEpiThreads);
        if (ok && warp == 4 && lane == 0 && !*abort_flag) {
            for (int c = 0; c < L::kChunks; ++c) tma_store_4d(&tmdQ, sQ + c * kTile, c * 64, t0, h, b);
            tma_store_commit();
            tma_store_wait_all();
        }
    }

    __syncwarp();
    if (*abort_flag) {
        const long long t_end = clock64() + (1LL << 19);
        while (clock64() < t_end) __nanosleep(256);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

// =============================================================================================
//                                    dK / dU / dV kernel
// =============================================================================================
template <int DH>
struct DwSmem {
    static constexpr int kChunks = (DH + 63) / 64;
    static constexpr uint32_t kWBytes = 3 * kChunks * kWChunk;  // [K;U] chunks then V chunks
    static constexpr uint32_t kOffWV = 2 * kChunks * kWChunk;
    static constexpr uint32_t kTokStage = 2 * kChunks * kTile;  // Q chunks then dO chunks
    static constexpr int kTokStages = 2;
    static constexpr uint32_t kOffW = 0;
    static constexpr uint32_t kOffTok = kOffW + kWBytes;
    static constexpr uint32_t kOffP = kOffTok + kTokStages * kTokStage;  // [dM | dN] : 2 x 16 KB
    static constexpr uint32_t kOffA = kOffP + 2 * kTile;                 // A : 16 KB
    static constexpr uint32_t kOffCtl = kOffA + kTile;
    static constexpr uint32_t kTotal = kOffCtl + 256 + 1024;
};

// The Q half and the dO half of a token stage, and the [dM|dN] tile and the A tile, have barriers of their
// own: each is needed by, and released after, a different MMA chain, and every cycle by which the next
// load or the next MMA can start earlier shortens the loop load -> recompute -> element-wise -> accumulate.
// S has two buffers in tensor memory, each with its own full/empty pair, so that every waiter sees every
// phase of the barrier it waits on (a one-bit parity cannot tell phase k from phase k+2).
enum { DW_WFULL = 0, DW_QFULL = 1, DW_GFULL = 3, DW_QEMPTY = 5, DW_GEMPTY = 7, DW_SFULL = 9, DW_SEMPTY = 11,
       DW_PFULL = 13, DW_AFULL = 14, DW_PEMPTY = 15, DW_AEMPTY = 16, DW_ACCFULL = 17, DW_DAEMPTY = 18, DW_BARS = 19 };

struct DwArgs {
    const float *R;
    long long r_sb, r_sh, r_ss;
    float *ws;  // [nsplit][3][Hkuv][I][DH] fp32 partial sums
    int S, E, De, G, B, Hkuv;
    int tiles_per_seq, tiles_total, tiles_per_split;
    // CTA -> (weight block, token-tile range).  Blocks [0, n_mixed) are split unevenly into a long part (launched first)
    // and a short part of `small_tiles` tiles (launched last); the others into `nsplit` equal parts, part by part.
    int nblk_j, n_blocks, nsplit, n_mixed, small_tiles;
    float s0, c;  // head_scaling; head_scaling * up_scaling * final_scaling
    WaitArgs wait;
};

template <int DH>
__global__ void __launch_bounds__(kThreads, 1)
bwd_dw_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
              const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmU,
              const __grid_constant__ CUtensorMap tmV, const DwArgs args) {
    using L = DwSmem<DH>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *gbase = smem_raw + (base - raw);
    const uint32_t sW = base + L::kOffW, sTok = base + L::kOffTok, sP = base + L::kOffP, sA = base + L::kOffA,
                   sBar = base + L::kOffCtl;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(gbase + L::kOffCtl + DW_BARS * 8);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(gbase + L::kOffCtl + DW_BARS * 8 + 4);
    auto bar = [&](int i) { return sBar + 8u * i; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int blk, split, tile_begin, tile_end;
    {
        const int cta = blockIdx.x, n_even = args.n_blocks - args.n_mixed;
        if (cta < args.n_mixed) {                               // long part of an unevenly split block
            blk = cta; split = 0; tile_begin = 0; tile_end = args.tiles_total - args.small_tiles;
        } else if (cta < args.n_mixed + n_even * args.nsplit) { // equal parts, part by part
            const int r = cta - args.n_mixed;
            split = r / n_even;
            blk = args.n_mixed + (r - split * n_even);
            tile_begin = split * args.tiles_per_split;
            tile_end = min(tile_begin + args.tiles_per_split, args.tiles_total);
        } else {                                                // short part of an unevenly split block
            blk = cta - (args.n_mixed + n_even * args.nsplit); split = 1;
            tile_begin = args.tiles_total - args.small_tiles; tile_end = args.tiles_total;
        }
    }
    const int hk = blk / args.nblk_j, jblk = blk - hk * args.nblk_j;
    const int e = (jblk * kBI) / args.De;
    const int ntiles = tile_end - tile_begin;  // >= 1 by construction of the plan
    const WaitCtl ctl{abort_flag, args.wait};
    constexpr int W = kKernelBwdDw * 100;
    // dV^T = sum_t dO^T A (d_h x 64, M = 128, N = 64) needs half the columns and three quarters of the tensor-pipe
    // time of dV = sum_t A^T dO (M = 64 runs at the M = 128 rate); it needs M = d_h = 128.
    constexpr bool kVt = DH == 128;
    // Columns: [dK;dU] at 0 (d_h wide), dV at 128 (64 wide transposed, else d_h wide), S buffers at 256 and 384, dA in
    // the gap at 192.  d_h = 96 leaves no gap (dV reaches column 224): it keeps one S buffer, with dA at 384.
    constexpr int kSB = DH == 96 ? 1 : 2;
    constexpr uint32_t kColKU = 0, kColV = 128, kColS = 256, kColdA = kSB == 2 ? 192 : 384;

    auto tile_coords = [&](int i, int &ts, int &hh, int &bb) {  // token tile i of this CTA -> (seq tile, head, batch)
        const int ti = tile_begin + i;
        ts = ti % args.tiles_per_seq;
        const int rest = ti / args.tiles_per_seq;
        hh = hk * args.G + rest % args.G;
        bb = rest / args.G;
    };

    if (threadIdx.x == 0) {
        *abort_flag = launch_aborted(args.wait);  // a CTA of this launch gave up: drain fast
        mbar_init(bar(DW_WFULL), 1);
        for (int s = 0; s < L::kTokStages; ++s) {
            mbar_init(bar(DW_QFULL + s), 1);
            mbar_init(bar(DW_GFULL + s), 1);
            mbar_init(bar(DW_QEMPTY + s), 1);
            mbar_init(bar(DW_GEMPTY + s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar(DW_SFULL + b), 1);
            mbar_init(bar(DW_SEMPTY + b), arrivals_of(kActThreads));
        }
        mbar_init(bar(DW_DAEMPTY), arrivals_of(kActThreads));
        mbar_init(bar(DW_PFULL), arrivals_of(kActThreads));
        mbar_init(bar(DW_AFULL), arrivals_of(kActThreads));
        mbar_init(bar(DW_PEMPTY), 1);
        mbar_init(bar(DW_AEMPTY), 1);
        mbar_init(bar(DW_ACCFULL), 1);
        fence_mbar_init();
    }
    if (warp == 1) tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const bool dead = *abort_flag != 0;

    if (dead) {
        // nothing: fall through to the teardown
    } else if (warp == 0) {
        if (lane == 0) {
            tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmdO); tma_prefetch_desc(&tmK);
            tma_prefetch_desc(&tmU); tma_prefetch_desc(&tmV);
            mbar_arrive_expect_tx(bar(DW_WFULL), L::kWBytes);
            const int row = jblk * kBI;
            for (int c = 0; c < L::kChunks; ++c) {
                tma_load_3d(sW + c * 2 * kWChunk, &tmK, bar(DW_WFULL), c * 64, row, hk);
                tma_load_3d(sW + c * 2 * kWChunk + kWChunk, &tmU, bar(DW_WFULL), c * 64, row, hk);
                tma_load_3d(sW + L::kOffWV + c * kWChunk, &tmV, bar(DW_WFULL), c * 64, row, hk);
            }
            int st = 0;
            uint32_t ph = 1;
            for (int i = 0; i < ntiles; ++i) {
                int ts, hh, bb;
                tile_coords(i, ts, hh, bb);
                const uint32_t d = sTok + st * L::kTokStage;
                if (!mbar_wait(bar(DW_QEMPTY + st), ph, ctl, W + 1)) break;
                const uint32_t fq = bar(DW_QFULL + st);
                mbar_arrive_expect_tx(fq, L::kTokStage / 2);
#pragma unroll
                for (int c = 0; c < L::kChunks; ++c) tma_load_4d(d + c * kTile, &tmQ, fq, c * 64, ts * kBT, hh, bb);
                if (!mbar_wait(bar(DW_GEMPTY + st), ph, ctl, W + 2)) break;
                const uint32_t fg = bar(DW_GFULL + st);
                mbar_arrive_expect_tx(fg, L::kTokStage / 2);
#pragma unroll
                for (int c = 0; c < L::kChunks; ++c)
                    tma_load_4d(d + (L::kChunks + c) * kTile, &tmdO, fg, c * 64, ts * kBT, hh, bb);
                if (++st == L::kTokStages) { st = 0; ph ^= 1; }
            }
        }
    } else if (warp == 1) {
        // MMA issuer 1: the recompute chain S = Q [K;U]^T, dA = dO V^T of each token tile.  The two
        // chains have their own issuing threads so that neither waits on the other's barriers and the
        // tensor pipe, which accepts MMAs only a few ahead of execution, is fed by whichever is ready.
        // Descriptors are built once and advanced by constants (16-byte units).
        if (lane == 0) {
            constexpr uint32_t idS = umma_idesc(128, 2 * kBI, false, false);
            constexpr uint32_t idA = umma_idesc(128, kBI, false, false);
            const uint64_t dQk0 = desc_kmajor(sTok), dGk0 = desc_kmajor(sTok + L::kChunks * kTile),
                           dKU = desc_kmajor(sW), dV = desc_kmajor(sW + L::kOffWV);
            constexpr uint64_t kTokStep = L::kTokStage >> 4;
            bool ok = mbar_wait(bar(DW_WFULL), 0, ctl, W + 3);
            int st = 0;
            uint32_t ph = 0;
            for (int i = 0; ok && i < ntiles; ++i) {
                if (!mbar_wait(bar(DW_QFULL + st), ph, ctl, W + 4)) break;
                const int sb = i % kSB;
                const uint32_t sph = (uint32_t)(i / kSB) & 1u;
                if (!mbar_wait(bar(DW_SEMPTY + sb), sph ^ 1, ctl, W + 5)) break;
                tc_fence_after();
                const uint64_t dq = dQk0 + st * kTokStep, dg = dGk0 + st * kTokStep;
#pragma unroll
                for (int k = 0; k < DH / 16; ++k) {
                    const int c = k >> 2, kk = k & 3;
                    umma_ss(tmem + kColS + sb * 2 * kBI, dq + ((c * kTile + kk * 32) >> 4),
                            dKU + ((c * 2 * kWChunk + kk * 32) >> 4), idS, k > 0 ? 1u : 0u);
                }
                if (!mbar_wait(bar(DW_GFULL + st), ph, ctl, W + 4)) break;
                if (!mbar_wait(bar(DW_DAEMPTY), (i & 1) ^ 1, ctl, W + 10)) break;
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < DH / 16; ++k) {
                    const int c = k >> 2, kk = k & 3;
                    umma_ss(tmem + kColdA, dg + ((c * kTile + kk * 32) >> 4), dV + ((c * kWChunk + kk * 32) >> 4), idA,
                            k > 0 ? 1u : 0u);
                }
                umma_commit(bar(DW_SFULL + sb));
                if (++st == L::kTokStages) { st = 0; ph ^= 1; }
            }
        }
    } else if (warp == 3) {
        // MMA issuer 2: the accumulation chain [dK;dU] += [dM|dN]^T Q, dV += A^T dO.
        if (lane == 0) {
            constexpr uint32_t idKU = umma_idesc(128, DH, true, true);
            constexpr uint32_t idV = kVt ? umma_idesc(128, kBI, true, true) : umma_idesc(64, DH, true, true);
            const uint64_t dQmn0 = desc_mnmajor(sTok, kTile), dGmn0 = desc_mnmajor(sTok + L::kChunks * kTile, kTile),
                           dPmn = desc_mnmajor(sP, kTile), dAmn = desc_mnmajor(sA, kTile);
            constexpr uint64_t kTokStep = L::kTokStage >> 4;
            int st = 0;
            bool ok = true;
            for (int i = 0; i < ntiles; ++i) {
                if (!mbar_wait(bar(DW_PFULL), i & 1, ctl, W + 6)) { ok = false; break; }
                tc_fence_after();
                const uint64_t dq = dQmn0 + st * kTokStep, dg = dGmn0 + st * kTokStep;
#pragma unroll
                for (int k = 0; k < kBT / 16; ++k)
                    umma_ss(tmem + kColKU, dPmn + k * 128, dq + k * 128, idKU, (i > 0 || k > 0) ? 1u : 0u);
                umma_commit(bar(DW_QEMPTY + st));  // Q of this stage and the [dM|dN] tile are free
                umma_commit(bar(DW_PEMPTY));
                if (!mbar_wait(bar(DW_AFULL), i & 1, ctl, W + 6)) { ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < kBT / 16; ++k) {
                    if (kVt) umma_ss(tmem + kColV, dg + k * 128, dAmn + k * 128, idV, (i > 0 || k > 0) ? 1u : 0u);
                    else umma_ss(tmem + kColV, dAmn + k * 128, dg + k * 128, idV, (i > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(bar(DW_GEMPTY + st));  // dO of this stage and the A tile are free
                umma_commit(bar(DW_AEMPTY));
                if (++st == L::kTokStages) st = 0;
            }
            if (ok) umma_commit(bar(DW_ACCFULL));
        }
    } else if (warp >= 4) {
        const int quarter = warp & 3, part = (warp - 4) >> 2, half = part;  // part: which kCols of the block's 64 columns
        const int row = quarter * 32 + lane;
        const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
        bool ok = true;
        const BwdConst kc = bwd_const(args.s0);
        // This row's routing weight for sub-network e, fetched one tile ahead.  The tile's (sequence tile, head, batch)
        // coordinates advance by counting, with no division in the loop.
        int c_ts, c_hh, c_bb;
        tile_coords(0, c_ts, c_hh, c_bb);
        int c_g = c_hh - hk * args.G;
        auto r_of_tile = [&]() {
            const int t = c_ts * kBT + row;
            return (t < args.S) ? __ldg(args.R + (long long)c_bb * args.r_sb + (long long)(hk * args.G + c_g) * args.r_sh +
                                        (long long)t * args.r_ss + e) : 0.f;
        };
        float r_next = r_of_tile();
        for (int i = 0; i < ntiles; ++i) {
            const float r = r_next;
            if (i + 1 < ntiles) {
                if (++c_ts == args.tiles_per_seq) {
                    c_ts = 0;
                    if (++c_g == args.G) { c_g = 0; ++c_bb; }
                }
                r_next = r_of_tile();
            }
            const int sb = i % kSB;
            if (!mbar_wait(bar(DW_SFULL + sb), (uint32_t)(i / kSB) & 1u, ctl, W + 7)) { ok = false; break; }
            tc_fence_after();
            uint32_t pm[kCols / 2], pn[kCols / 2], pa[kCols / 2], da[kCols];
            // dA first: its single buffer goes straight back
            if (kCols == 32) tmem_ld32_sync(lane_base + kColdA + part * kCols, da);
            else tmem_ld16_sync(lane_base + kColdA + part * kCols, da);
            tc_fence_before();
            warp_arrive(bar(DW_DAEMPTY));
            const f32x2 r2 = f2_pack(args.c * r, args.c * r);
            const uint32_t colS = kColS + sb * 2 * kBI;
#pragma unroll
            for (int sub = 0; sub < kSubs; ++sub) {
                uint32_t m[16], n[16];
                const uint32_t c = part * kCols + sub * 16;
                tmem_ld16x2_sync(lane_base + colS + c, lane_base + colS + kBI + c, m, n);
                if (sub == kSubs - 1) {   // S is in registers: the buffer can take the tile after next
                    tc_fence_before();
                    warp_arrive(bar(DW_SEMPTY + sb));
                }
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const BwdPair x = bwd_pair(f2_pack_bits(m[2 * q], m[2 * q + 1]), f2_pack_bits(n[2 * q], n[2 * q + 1]),
                                               f2_pack_bits(da[sub * 16 + 2 * q], da[sub * 16 + 2 * q + 1]), r2, kc);
                    pm[sub * 8 + q] = f2_to_bf16x2(x.dm);
                    pn[sub * 8 + q] = f2_to_bf16x2(x.dn);
                    pa[sub * 8 + q] = f2_to_bf16x2(f2_mul(x.sn, r2));
                }
            }
            if (!mbar_wait(bar(DW_PEMPTY), (i & 1) ^ 1, ctl, W + 8)) { ok = false; break; }
#pragma unroll
            for (int q = 0; q < kCols / 8; ++q) {
                const uint32_t off = sw128_offset(row, part * (kCols / 8) + q);
                st_shared_v4(sP + off, pm[4 * q], pm[4 * q + 1], pm[4 * q + 2], pm[4 * q + 3]);
                st_shared_v4(sP + kTile + off, pn[4 * q], pn[4 * q + 1], pn[4 * q + 2], pn[4 * q + 3]);
            }
            fence_async_smem();
            warp_arrive(bar(DW_PFULL));
            if (!mbar_wait(bar(DW_AEMPTY), (i & 1) ^ 1, ctl, W + 8)) { ok = false; break; }
#pragma unroll
            for (int q = 0; q < kCols / 8; ++q)
                st_shared_v4(sA + sw128_offset(row, part * (kCols / 8) + q), pa[4 * q], pa[4 * q + 1], pa[4 * q + 2], pa[4 * q + 3]);
            fence_async_smem();
            warp_arrive(bar(DW_AFULL));
        }
        if (part >= 2) ok = false;  // the accumulators are written out by the warps of parts 0 and 1
        if (ok) ok = mbar_wait(bar(DW_ACCFULL), 0, ctl, W + 9);
        if (ok) {
            tc_fence_after();
            // fp32 partial sums -> workspace[split][which][hk][row][DH]
            const long long I = (long long)args.E * args.De;
            const long long plane = (long long)args.Hkuv * I * DH;
            float *wsb = args.ws + (long long)split * 3 * plane + ((long long)hk * I + (long long)jblk * kBI) * DH;
            constexpr int kColsPerHalf = DH / 2;
            const int c0 = half * kColsPerHalf;
            {   // [dK;dU]: lane = row of the stacked block (0-63 dK, 64-127 dU)
                float *dst = wsb + (row < kBI ? 0 : plane) + (long long)(row & (kBI - 1)) * DH + c0;
#pragma unroll
                for (int g = 0; g < kColsPerHalf / 16; ++g) {
                    uint32_t o[16];
                    tmem_ld16_sync(lane_base + kColKU + c0 + g * 16, o);
#pragma unroll
                    for (int v = 0; v < 4; ++v)
                        *reinterpret_cast<float4 *>(dst + g * 16 + v * 4) =
                            make_float4(__uint_as_float(o[4 * v]), __uint_as_float(o[4 * v + 1]),
                                        __uint_as_float(o[4 * v + 2]), __uint_as_float(o[4 * v + 3]));
                }
            }
            if (kVt) {  // dV^T: lane = column d of dV, tensor-memory column = row of the block; a warp stores 32 consecutive floats per row
                float *dst = wsb + 2 * plane + row;
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    uint32_t o[16];
                    tmem_ld16_sync(lane_base + kColV + half * 32 + g * 16, o);
#pragma unroll
                    for (int v = 0; v < 16; ++v) dst[(long long)(half * 32 + g * 16 + v) * DH] = __uint_as_float(o[v]);
                }
            } else {    // dV (M = 64 accumulator): row r lives in TMEM lane 32*(r/16) + r%16
                float *dst = wsb + 2 * plane + (long long)(quarter * 16 + (lane & 15)) * DH + c0;
#pragma unroll
                for (int g = 0; g < kColsPerHalf / 16; ++g) {
                    uint32_t o[16];
                    tmem_ld16_sync(lane_base + kColV + c0 + g * 16, o);
                    if (lane < 16) {
#pragma unroll
                        for (int v = 0; v < 4; ++v)
                            *reinterpret_cast<float4 *>(dst + g * 16 + v * 4) =
                                make_float4(__uint_as_float(o[4 * v]), __uint_as_float(o[4 * v + 1]),
                                            __uint_as_float(o[4 * v + 2]), __uint_as_float(o[4 * v + 3]));
                    }
                }
            }
            tc_fence_before();
        }
    }

    __syncwarp();
    if (*abort_flag) {
        const long long t_end = clock64() + (1LL << 19);
        while (clock64() < t_end) __nanosleep(256);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

// Sum the token-axis splits in index order and write bf16 gradients (4 elements per thread).
struct ReduceArgs {
    const float *ws;
    __nv_bfloat16 *out[3];
    long long s_head[3], s_row[3];
    long long plane;  // Hkuv * I * DH
    int nsplit, I, DH;
};
__global__ void __launch_bounds__(256) dw_reduce_kernel(const ReduceArgs a) {
    const long long n4 = 3 * a.plane / 4;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n4;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long el = idx * 4;
        float4 acc = *reinterpret_cast<const float4 *>(a.ws + el);
        for (int s = 1; s < a.nsplit; ++s) {
            const float4 v = *reinterpret_cast<const float4 *>(a.ws + (long long)s * 3 * a.plane + el);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        const int which = (int)(el / a.plane);
        const long long rem = el - (long long)which * a.plane;
        const int c = (int)(rem % a.DH);
        const long long rowi = rem / a.DH;
        const int r = (int)(rowi % a.I), hk = (int)(rowi / a.I);
        __nv_bfloat16 *o = a.out[which] + hk * a.s_head[which] + r * a.s_row[which] + c;
        uint2 packed = make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
        *reinterpret_cast<uint2 *>(o) = packed;
    }
}

int choose_nsplit(long long items, int tiles_total, int num_sms) {
    int best = 1;
    double best_eff = 0.0;
    for (int ns = 1; ns <= 16 && ns <= tiles_total; ++ns) {
        const long long ctas = items * ns;
        const long long waves = (ctas + num_sms - 1) / num_sms;
        const double eff = (double)ctas / (double)(waves * num_sms);
        if (eff > best_eff + 1e-9) { best_eff = eff; best = ns; }
        if (eff >= 0.9) return ns;
    }
    return best;
}

struct DwPlan {
    int tiles_per_seq, tiles_total, nsplit, tiles_per_split;
    int n_mixed, small_tiles;   // uneven split of the first n_mixed blocks (two-way splits only), else 0
};

// Time at which the last of `jobs` (durations, in launch order) ends when each goes to the SM that frees up first.
double list_schedule(const std::vector<double> &jobs, int num_sms) {
    std::priority_queue<double, std::vector<double>, std::greater<double>> sm;
    for (int i = 0; i < num_sms; ++i) sm.push(0.0);
    double end = 0.0;
    for (double j : jobs) {
        const double t = sm.top() + j;
        sm.pop();
        sm.push(t);
        if (t > end) end = t;
    }
    return end;
}

// With a two-way split the CTAs are equal and their last wave is partly empty (704 CTAs on 148 SMs: the fifth wave is
// 76 % full, 5 % of the kernel).  Splitting some blocks unevenly -- long parts launched first, short parts last, the
// equal halves of the other blocks in between -- lets the short parts fill the SMs the last wave would leave idle.
// The split point and the number of such blocks are found by simulating the launch order for a few candidates; a CTA's
// fixed cost (weights in, accumulators out) is taken as two token tiles.  The partial sums still number two per
// block, so the reduction and the workspace do not change.
void plan_uneven(DwPlan &p, long long items, int num_sms) {
    p.n_mixed = p.small_tiles = 0;
    if (p.nsplit != 2 || items > 2048 || p.tiles_total < 32) return;
    const double ovh = 2.0;
    const int T = p.tiles_total, half = p.tiles_per_split;
    auto makespan = [&](int nmix, int small) {
        std::vector<double> jobs;
        jobs.reserve((size_t)(2 * items));
        for (int i = 0; i < nmix; ++i) jobs.push_back(T - small + ovh);
        for (long long i = 0; i < items - nmix; ++i) jobs.push_back(half + ovh);
        for (long long i = 0; i < items - nmix; ++i) jobs.push_back(T - half + ovh);
        for (int i = 0; i < nmix; ++i) jobs.push_back(small + ovh);
        return list_schedule(jobs, num_sms);
    };
    const double base = makespan(0, 0);
    double best = base;
    const int step_small = T / 32 > 1 ? T / 32 : 1, step_mix = num_sms / 4 > 1 ? num_sms / 4 : 1;
    for (int small = step_small; small < half; small += step_small)
        for (int nmix = step_mix; nmix <= items; nmix += step_mix) {
            const double m = makespan(nmix, small);
            if (m < best - 1e-9) { best = m; p.n_mixed = nmix; p.small_tiles = small; }
        }
    if (best > 0.985 * base) p.n_mixed = p.small_tiles = 0;   // not worth a different launch order
}

DwPlan dw_plan(const flashmhf_dims &d, int num_sms) {
    struct Key { long long items; int tiles_per_seq, tiles_total, num_sms; };
    struct Entry { Key k; DwPlan p; };
    static std::mutex mu;
    static std::vector<Entry> cache;
    const int G = d.H / d.Hkuv;
    const long long items = (long long)d.Hkuv * ((long long)d.E * d.De / kBI);
    const Key key{items, (d.S + kBT - 1) / kBT, ((d.S + kBT - 1) / kBT) * G * d.B, num_sms};
    std::lock_guard<std::mutex> lk(mu);
    for (const Entry &e : cache)
        if (e.k.items == key.items && e.k.tiles_per_seq == key.tiles_per_seq && e.k.tiles_total == key.tiles_total &&
            e.k.num_sms == key.num_sms)
            return e.p;
    DwPlan p;
    p.tiles_per_seq = key.tiles_per_seq;
    p.tiles_total = key.tiles_total;
    const int ns = choose_nsplit(items, p.tiles_total, num_sms);
    p.tiles_per_split = (p.tiles_total + ns - 1) / ns;
    p.nsplit = (p.tiles_total + p.tiles_per_split - 1) / p.tiles_per_split;  // no empty split
    plan_uneven(p, items, num_sms);
    if (cache.size() < 256) cache.push_back(Entry{key, p});
    return p;
}

template <int DH>
int launch_bwd(const flashmhf_bwd_params &p, cudaStream_t st, int *n_launch) {
    const flashmhf_dims &d = p.d;
    const DeviceCtl *dc = device_ctl();
    if (!dc) return FLASHMHF_ERR_CUDA;
    const bool want_inputs = (p.parts & FLASHMHF_BWD_INPUTS) != 0, want_weights = (p.parts & FLASHMHF_BWD_WEIGHTS) != 0;
    CUtensorMap tmQ, tmdO, tmK, tmU, tmV, tmdQ;
    int rc;
    if ((rc = encode_act_map(&tmQ, p.Q, d, kBT)) != 0) return rc;
    if ((rc = encode_act_map(&tmdO, p.dO, d, kBT)) != 0) return rc;
    if ((rc = encode_weight_map(&tmK, p.K, d, kBI)) != 0) return rc;
    if ((rc = encode_weight_map(&tmU, p.U, d, kBI)) != 0) return rc;
    if ((rc = encode_weight_map(&tmV, p.V, d, kBI)) != 0) return rc;
    if (want_inputs && (rc = encode_act_map(&tmdQ, p.dQ, d, kBT)) != 0) return rc;
    if (want_weights)
        for (const flashmhf_tensor *t : {&p.dK, &p.dU, &p.dV}) {
            if (d.E > 1 && t->stride[1] != (int64_t)d.De * t->stride[2]) return FLASHMHF_ERR_BAD_STRIDE;
            if (t->stride[2] % 4 != 0 || t->stride[0] % 4 != 0) return FLASHMHF_ERR_BAD_STRIDE;
        }
    cudaError_t e;
    {  // the attribute is per device and per kernel: set once for each pair
        static std::atomic<bool> done[64];
        if (!done[dc->device].load(std::memory_order_acquire)) {
            e = cudaFuncSetAttribute(bwd_dq_kernel<DH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DqSmem<DH>::kTotal);
            if (e == cudaSuccess)
                e = cudaFuncSetAttribute(bwd_dw_kernel<DH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DwSmem<DH>::kTotal);
            if (e != cudaSuccess) { set_cuda_error(e, "cudaFuncSetAttribute(bwd kernels)"); return FLASHMHF_ERR_CUDA; }
            done[dc->device].store(true, std::memory_order_release);
        }
    }
    const int G = d.H / d.Hkuv;
    const float s0 = p.scale.head_scaling, c = p.scale.head_scaling * p.scale.up_scaling * p.scale.final_scaling;

    // Weight gradients first: in data-parallel training their all-reduce can then start while dQ/dR still run.
    if (want_weights) {
        const DwPlan pl = dw_plan(d, dc->num_sms);
        DwArgs wa{static_cast<const float *>(p.R.ptr), p.R.stride[0], p.R.stride[1], p.R.stride[2],
                  static_cast<float *>(p.workspace), d.S, d.E, d.De, G, d.B, d.Hkuv,
                  pl.tiles_per_seq, pl.tiles_total, pl.tiles_per_split,
                  d.E * d.De / kBI, d.Hkuv * (d.E * d.De / kBI), pl.nsplit, pl.n_mixed, pl.small_tiles, s0, c, wait_args(dc)};
        const long long ctas = (long long)wa.n_blocks * pl.nsplit;
        if (ctas > 0x7fffffffLL) return FLASHMHF_ERR_BAD_SHAPE;
        dim3 gw((unsigned)ctas);
        prof_mark(st, kMarkStart);
        bwd_dw_kernel<DH><<<gw, kThreads, DwSmem<DH>::kTotal, st>>>(tmQ, tmdO, tmK, tmU, tmV, wa);
        prof_mark(st, kMarkBwdDw);
        *n_launch += 1;
        if ((e = cudaGetLastError()) != cudaSuccess) { set_cuda_error(e, "bwd_dw_kernel launch"); return FLASHMHF_ERR_CUDA; }

        ReduceArgs ra;
        ra.ws = static_cast<const float *>(p.workspace);
        const flashmhf_tensor *outs[3] = {&p.dK, &p.dU, &p.dV};
        for (int i = 0; i < 3; ++i) {
            ra.out[i] = static_cast<__nv_bfloat16 *>(outs[i]->ptr);
            ra.s_head[i] = outs[i]->stride[0];
            ra.s_row[i] = outs[i]->stride[2];
        }
        ra.I = d.E * d.De;
        ra.DH = DH;
        ra.plane = (long long)d.Hkuv * ra.I * DH;
        ra.nsplit = pl.nsplit;
        const long long n4 = 3 * ra.plane / 4, cap = (long long)dc->num_sms * 8;
        const int blocks = (int)((n4 + 255) / 256 < cap ? (n4 + 255) / 256 : cap);
        dw_reduce_kernel<<<blocks, 256, 0, st>>>(ra);
        prof_mark(st, kMarkBwdReduce);
        *n_launch += 1;
        if ((e = cudaGetLastError()) != cudaSuccess) { set_cuda_error(e, "dw_reduce_kernel launch"); return FLASHMHF_ERR_CUDA; }
    }

    if (want_inputs) {
        DqArgs qa{static_cast<const float *>(p.R.ptr), p.R.stride[0], p.R.stride[1], p.R.stride[2],
                  static_cast<float *>(p.dR.ptr), p.dR.stride[0], p.dR.stride[1], p.dR.stride[2],
                  d.S, d.E, d.De, G, s0, c, wait_args(dc)};
        dim3 gq((d.S + kBT - 1) / kBT, d.H, d.B);
        prof_mark(st, kMarkStart);
        bwd_dq_kernel<DH><<<gq, kThreads, DqSmem<DH>::kTotal, st>>>(tmQ, tmdO, tmK, tmU, tmV, tmdQ, qa);
        prof_mark(st, kMarkBwdDq);
        *n_launch += 1;
        if ((e = cudaGetLastError()) != cudaSuccess) { set_cuda_error(e, "bwd_dq_kernel launch"); return FLASHMHF_ERR_CUDA; }
    }
    return FLASHMHF_OK;
}

}  // namespace

size_t tc_backward_workspace_bytes(const flashmhf_dims &d) {
    const DeviceCtl *dc = device_ctl();
    const DwPlan pl = dw_plan(d, dc ? dc->num_sms : 148);
    return (size_t)pl.nsplit * 3 * (size_t)d.Hkuv * (size_t)d.E * d.De * d.Dh * sizeof(float);
}

// ---------------------------------------------------------------------------------------------
// Built-in scratch for flashmhf_backward_static_scratch: the split partial sums of dK/dU/dV live in
// this file-scope device array instead of a caller-provided workspace.  One copy per GPU that loads
// the library, held until the process exits.  The dK/dU/dV kernel writes every partial it later
// reads, so nothing here has to start at zero.
constexpr size_t kStaticScratchBytes = FLASHMHF_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_scratch_mu;
void *g_scratch_addr[kMaxDevices] = {nullptr};

// In host code `g_static_scratch` is only a handle for the symbol, not a device address: the
// address is looked up once per device, with that device current, and cached.
int static_scratch_ptr(void **out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        set_cuda_error(e, "cudaGetDevice (static scratch)");
        return FLASHMHF_ERR_CUDA;
    }
    std::lock_guard<std::mutex> lk(g_scratch_mu);
    if (!g_scratch_addr[dev]) {
        void *ptr = nullptr;
        e = cudaGetSymbolAddress((void **)&ptr, g_static_scratch);
        if (e != cudaSuccess || !ptr) {
            set_cuda_error(e, "cudaGetSymbolAddress(g_static_scratch)");
            return FLASHMHF_ERR_CUDA;
        }
        g_scratch_addr[dev] = ptr;
    }
    *out = g_scratch_addr[dev];
    return FLASHMHF_OK;
}
}  // namespace

int tc_backward_static_scratch(const flashmhf_bwd_params &p, cudaStream_t st, int *n_launch) {
    if (tc_backward_workspace_bytes(p.d) > kStaticScratchBytes) return FLASHMHF_ERR_SCRATCH_LIMIT;
    void *ptr = nullptr;
    const int rc = static_scratch_ptr(&ptr);
    if (rc != FLASHMHF_OK) return rc;
    flashmhf_bwd_params q = p;
    q.workspace = ptr;
    q.workspace_bytes = kStaticScratchBytes;
    return tc_backward(q, st, n_launch);
}

int tc_backward(const flashmhf_bwd_params &p, cudaStream_t st, int *n_launch) {
    switch (p.d.Dh) {
        case 64: return launch_bwd<64>(p, st, n_launch);
        case 96: return launch_bwd<96>(p, st, n_launch);
        case 128: return launch_bwd<128>(p, st, n_launch);
        default: return FLASHMHF_ERR_BAD_SHAPE;
    }
}

}  // namespace fmhf
