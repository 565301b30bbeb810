// Forward kernel, bf16, sm_100a:  O = sum_e R_e * ((SiLU(Q K_e^T) * (Q U_e^T)) V_e).
//
// One CTA owns one tile of 128 token rows of one (batch, head).  Its Q tile is loaded once; the
// weights of the head stream through shared-memory rings, 64 intermediate rows (one "block": 64
// rows of K_e, U_e and V_e) at a time.  Per block the tensor core computes
//     S = Q [K_blk; U_blk]^T      (128 x 128, one MMA chain, fp32 in tensor memory: M | N)
// an activation warpgroup reads S, forms A = bf16(SiLU(M) * N * R_e) in registers and writes it
// back into tensor memory over the first 32 columns of the same S buffer (two bf16 per column), and
// the tensor core accumulates, with A read from tensor memory and V from shared memory,
//     O += A V_blk                (128 x d_h, fp32 in tensor memory, over all blocks of all e)
// so the [T, E*d_e] intermediate never leaves the SM and A never touches shared memory.
//
// Pipeline.  The hand-off from an MMA to the warps that consume its result costs several hundred
// cycles (commit -> mbarrier -> wake-up) and the tensor pipe accepts MMAs only a few ahead of their
// execution, so (a) three S buffers keep three blocks in flight, (b) the two MMA chains are issued
// by two different threads -- one runs ahead with S = Q [K;U]^T, the other follows with O += A V --
// so that neither waits on the other's barriers, and (c) the two activation warpgroups own
// alternate blocks (even / odd), so the load/store phases of one overlap the arithmetic of the other.
//
// Warp roles (384 threads): warp 0 TMA producer, warps 1-2 MMA issuers for S (even / odd blocks;
// warp 1 owns tensor memory), warp 3 MMA issuer for O, warps 4-7 activation warpgroup 0,
// warps 8-11 activation warpgroup 1 (warp % 4 = TMEM lane quarter = 32 token rows; one thread = one
// token row of a block).
//
// Tensor memory (512 columns): O at [0, d_h), S buffers at [128, 256), [256, 384), [384, 512).
#include <atomic>

#include "kernels.h"
#include "tc_common.cuh"
#include "tensormap.cuh"

namespace fmhf {
namespace {

constexpr int kBT = 128;  // token rows per tile
constexpr int kBI = 64;   // intermediate rows per block
constexpr int kDepth = 3; // S buffers in tensor memory = blocks in flight
constexpr int kRing = 4;  // shared-memory stages of the [K;U] ring and of the V ring
constexpr int kThreads = 384;
constexpr int kGroupThreads = 128;  // one activation warpgroup
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColO = 0, kColS0 = 128, kColSStride = 128;

template <int DH>
struct FwdSmem {
    static constexpr int kChunks = (DH + 63) / 64;              // 64-column SW128 chunks per row of d_h
    static constexpr uint32_t kQBytes = kChunks * kBT * 128;    // Q tile (also the O staging tile)
    static constexpr uint32_t kWChunk = kBI * 128;              // one 64-row x 64-col weight chunk
    static constexpr uint32_t kKUStage = 2 * kChunks * kWChunk; // per chunk: K rows then U rows = one 128-row K-major tile
    static constexpr uint32_t kVStage = kChunks * kWChunk;
    // offsets from the 1024-aligned base
    static constexpr uint32_t kOffQ = 0;
    static constexpr uint32_t kOffKU = kOffQ + kQBytes;
    static constexpr uint32_t kOffV = kOffKU + kRing * kKUStage;
    static constexpr uint32_t kOffBar = kOffV + kRing * kVStage;
    static constexpr uint32_t kTotal = kOffBar + 320 + 1024;  // + barriers/control + alignment slack
};

// barrier slots (8 bytes each) inside the control area
// SFULL: S computed; AFULL: A written over it; SFREE: O += A V done, buffer reusable
// The three S-buffer barriers exist in 2 * kDepth copies, indexed by block % (2 * kDepth).  Blocks of
// even and odd index are handled by different threads (two S issuers, two activation warpgroups), so
// with one barrier per buffer a waiter would see only every other phase of it, and a one-bit phase
// parity cannot tell "two phases behind" from "done".  With 2 * kDepth barriers every barrier has one
// fixed waiter that observes each of its phases.
enum { BAR_Q = 0, BAR_KUFULL = 1, BAR_KUEMPTY = 5, BAR_VFULL = 9, BAR_VEMPTY = 13, BAR_SFULL = 17, BAR_AFULL = 23,
       BAR_SFREE = 29, BAR_OFULL = 35, BAR_COUNT = 36 };
constexpr int kSBars = 2 * kDepth;

struct FwdArgs {
    const float *R;
    long long r_sb, r_sh, r_ss;
    int S, E, De, G;
    // Split of the intermediate dimension over CTAs (short token counts, e.g. decode): CTA x handles
    // blocks [isplit * blocks_per_split, ...) of tile x / nsplit and writes an fp32 partial O.
    int nsplit, blocks_per_split;
    float *part;           // [nsplit][B][H][S][DH] fp32, used when nsplit > 1
    int H;
    float half_s0;  // 0.5 * head_scaling: tanh argument scale, sigmoid(s0 m) = 0.5 + 0.5 tanh(0.5 s0 m)
    float c;        // head_scaling * up_scaling * final_scaling, folded into the routing weight
    WaitArgs wait;
};

// Ring position of block j in a ring of N slots: slot j % N and the parity of its lap.
template <int N>
struct RingPos {
    int slot = 0;
    uint32_t lap = 0;
    __device__ __forceinline__ void advance(int by) {
        slot += by;
        if (slot >= N) { slot -= N; lap ^= 1; }
    }
};

template <int DH>
__global__ void __launch_bounds__(kThreads, 1)
fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
           const __grid_constant__ CUtensorMap tmU, const __grid_constant__ CUtensorMap tmV,
           const __grid_constant__ CUtensorMap tmO, const FwdArgs args) {
    using L = FwdSmem<DH>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *gbase = smem_raw + (base - raw);
    const uint32_t sQ = base + L::kOffQ, sKU = base + L::kOffKU, sV = base + L::kOffV, sBar = base + L::kOffBar;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(gbase + L::kOffBar + BAR_COUNT * 8);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(gbase + L::kOffBar + BAR_COUNT * 8 + 4);
    auto bar = [&](int i) { return sBar + 8u * i; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x / args.nsplit, isplit = blockIdx.x - tile * args.nsplit;
    const int t0 = tile * kBT, h = blockIdx.y, b = blockIdx.z, hk = h / args.G;
    const int blocks_per_e = args.De / kBI;
    const int j0 = isplit * args.blocks_per_split;                          // first block of this CTA
    const int nblk = min(args.E * blocks_per_e - j0, args.blocks_per_split);  // blocks of this CTA (>= 1)
    const WaitCtl ctl{abort_flag, args.wait};
    constexpr int W = kKernelFwd * 100;

    if (threadIdx.x == 0) {
        *abort_flag = launch_aborted(args.wait);  // a CTA of this launch gave up: drain fast
        mbar_init(bar(BAR_Q), 1);
        for (int i = 0; i < kRing; ++i) {
            mbar_init(bar(BAR_KUFULL + i), 1);
            mbar_init(bar(BAR_KUEMPTY + i), 1);
            mbar_init(bar(BAR_VFULL + i), 1);
            mbar_init(bar(BAR_VEMPTY + i), 1);
        }
        for (int i = 0; i < kSBars; ++i) {
            mbar_init(bar(BAR_SFULL + i), 1);
            mbar_init(bar(BAR_AFULL + i), arrivals_of(kGroupThreads));
            mbar_init(bar(BAR_SFREE + i), 1);
        }
        mbar_init(bar(BAR_OFULL), 1);
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
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            tma_prefetch_desc(&tmQ);
            tma_prefetch_desc(&tmK);
            tma_prefetch_desc(&tmU);
            tma_prefetch_desc(&tmV);
            mbar_arrive_expect_tx(bar(BAR_Q), L::kQBytes);
            for (int c = 0; c < L::kChunks; ++c) tma_load_4d(sQ + c * (kBT * 128), &tmQ, bar(BAR_Q), c * 64, t0, h, b);
            // [K;U] of block j, then V of block j-2: V is consumed about two blocks later than K and U of
            // the same block, so with this lag the producer never waits on the V ring while a [K;U]
            // stage is free.
            RingPos<kRing> pk, pv;
            for (int j = 0; j < nblk + 2; ++j) {
                if (j < nblk) {
                    if (!mbar_wait(bar(BAR_KUEMPTY + pk.slot), pk.lap ^ 1, ctl, W + 1)) break;
                    const uint32_t fku = bar(BAR_KUFULL + pk.slot), dku = sKU + pk.slot * L::kKUStage;
                    mbar_arrive_expect_tx(fku, L::kKUStage);
#pragma unroll
                    for (int c = 0; c < L::kChunks; ++c) {
                        tma_load_3d(dku + c * 2 * L::kWChunk, &tmK, fku, c * 64, (j0 + j) * kBI, hk);
                        tma_load_3d(dku + c * 2 * L::kWChunk + L::kWChunk, &tmU, fku, c * 64, (j0 + j) * kBI, hk);
                    }
                    pk.advance(1);
                }
                if (j >= 2) {
                    if (!mbar_wait(bar(BAR_VEMPTY + pv.slot), pv.lap ^ 1, ctl, W + 2)) break;
                    const uint32_t fv = bar(BAR_VFULL + pv.slot), dv = sV + pv.slot * L::kVStage;
                    mbar_arrive_expect_tx(fv, L::kVStage);
#pragma unroll
                    for (int c = 0; c < L::kChunks; ++c)
                        tma_load_3d(dv + c * L::kWChunk, &tmV, fv, c * 64, (j0 + j - 2) * kBI, hk);
                    pv.advance(1);
                }
            }
        }
    } else if (warp == 1 || warp == 2) {
        // ------------------------------------------------------------------ MMA issuers for S = Q [K;U]^T
        // Two threads (warp 1: even blocks, warp 2: odd blocks): while one is between batches -- barrier
        // polls, commits -- the other keeps the tensor pipe fed.  Blocks are independent (own S buffer).
        // One thread issues the chain, so its instruction stream is kept minimal: descriptors are built
        // once and advanced by adding constants (the address field counts 16-byte units).
        if (lane == 0) {
            constexpr uint32_t idesc1 = umma_idesc(128, 2 * kBI, false, false);
            const uint64_t dQ = desc_kmajor(sQ), dKU0 = desc_kmajor(sKU);
            constexpr uint64_t kKUStep = L::kKUStage >> 4;
            const int first = warp - 1;
            bool ok = mbar_wait(bar(BAR_Q), 0, ctl, W + 3);
            RingPos<kRing> pw;   // [K;U] stage of block j
            RingPos<kSBars> ps;  // barrier set of block j; its S buffer is ps.slot % kDepth
            RingPos<kSBars> pf;  // barrier set of block j - kDepth, the previous user of that buffer
            pf.lap = 1;          // so that the lap parity is 0 once j - kDepth reaches 0
            pw.advance(first);
            ps.advance(first);
            pf.advance(first + kDepth);
            for (int j = first; ok && j < nblk; j += 2) {
                if (!mbar_wait(bar(BAR_KUFULL + pw.slot), pw.lap, ctl, W + 4)) break;
                if (j >= kDepth && !mbar_wait(bar(BAR_SFREE + pf.slot), pf.lap, ctl, W + 5)) break;
                tc_fence_after();
                const uint64_t dku = dKU0 + pw.slot * kKUStep;
                const uint32_t tS = tmem + kColS0 + (ps.slot >= kDepth ? ps.slot - kDepth : ps.slot) * kColSStride;
#pragma unroll
                for (int k = 0; k < DH / 16; ++k) {
                    const int c = k >> 2, kk = k & 3;
                    umma_ss(tS, dQ + ((c * (kBT * 128) + kk * 32) >> 4), dku + ((c * 2 * L::kWChunk + kk * 32) >> 4),
                            idesc1, k > 0 ? 1u : 0u);
                }
                umma_commit(bar(BAR_KUEMPTY + pw.slot));
                umma_commit(bar(BAR_SFULL + ps.slot));
                pw.advance(2);
                ps.advance(2);
                pf.advance(2);
            }
        }
    } else if (warp == 3) {
        // ------------------------------------------------------------------ MMA issuer 2: O += A V
        // A comes from tensor memory (the first 32 columns of the block's S buffer), V from shared
        // memory as an MN-major operand.
        if (lane == 0) {
            constexpr uint32_t idesc2 = umma_idesc(128, DH, false, true);
            const uint64_t dV0 = desc_mnmajor(sV, L::kWChunk);
            constexpr uint64_t kVStep = L::kVStage >> 4;
            RingPos<kRing> pw;
            RingPos<kSBars> ps;
            bool ok = true;
            for (int j = 0; j < nblk; ++j) {
                if (!mbar_wait(bar(BAR_VFULL + pw.slot), pw.lap, ctl, W + 6)) { ok = false; break; }
                if (!mbar_wait(bar(BAR_AFULL + ps.slot), ps.lap, ctl, W + 7)) { ok = false; break; }
                tc_fence_after();
                const uint64_t dv = dV0 + pw.slot * kVStep;
                const uint32_t tA = tmem + kColS0 + (ps.slot >= kDepth ? ps.slot - kDepth : ps.slot) * kColSStride;
#pragma unroll
                for (int k = 0; k < kBI / 16; ++k)
                    umma_ts(tmem + kColO, tA + k * 8, dv + k * 128, idesc2, (j > 0 || k > 0) ? 1u : 0u);
                umma_commit(bar(BAR_VEMPTY + pw.slot));
                umma_commit(bar(BAR_SFREE + ps.slot));
                pw.advance(1);
                ps.advance(1);
            }
            if (ok) umma_commit(bar(BAR_OFULL));
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------------ activation + epilogue
        const int quarter = warp & 3, group = (warp - 4) >> 2;  // group 0: even blocks, group 1: odd blocks
        const int row = quarter * 32 + lane;
        const int t = t0 + row;
        const bool in_range = t < args.S;
        const float *rrow = args.R + (long long)b * args.r_sb + (long long)h * args.r_sh + (long long)t * args.r_ss;
        const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
        bool ok = true;
        const f32x2 half_s0 = f2_pack(args.half_s0, args.half_s0);
        // sub-network of this group's current block and position inside it; routing weight fetched a block ahead
        int e = (j0 + group) / blocks_per_e, in_e = (j0 + group) - e * blocks_per_e;
        float r_cur = (in_range && e < args.E) ? __ldg(rrow + e) : 0.f;
        RingPos<kSBars> p;
        p.advance(group);
        for (int j = group; j < nblk; j += 2) {
            int e_nb = e, in_nb = in_e + 2;  // where this group's next block lies
            while (in_nb >= blocks_per_e) { in_nb -= blocks_per_e; ++e_nb; }
            const float r_nb = (e_nb != e && in_range && e_nb < args.E) ? __ldg(rrow + e_nb) : r_cur;
            const float hr = 0.5f * args.c * r_cur;
            const f32x2 half_r = f2_pack(hr, hr);
            if (!mbar_wait(bar(BAR_SFULL + p.slot), p.lap, ctl, W + 8)) { ok = false; break; }
            tc_fence_after();
            const uint32_t ts = lane_base + kColS0 + (p.slot >= kDepth ? p.slot - kDepth : p.slot) * kColSStride;
            uint32_t a[32];  // 64 bf16 of this row of A
#pragma unroll
            for (int part = 0; part < 2; ++part) {
                uint32_t m[32], n[32];
                tmem_ld32x2_sync(ts + part * 32, ts + kBI + part * 32, m, n);
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    a[part * 16 + i] = fwd_act_pair(f2_pack_bits(m[2 * i], m[2 * i + 1]),
                                                    f2_pack_bits(n[2 * i], n[2 * i + 1]), half_r, half_s0);
            }
            tmem_st32(ts, a);  // over M[0:32] of this buffer, which is in registers by now
            tmem_st_wait();
            tc_fence_before();
            warp_arrive(bar(BAR_AFULL + p.slot));
            p.advance(2);
            r_cur = r_nb;
            e = e_nb;
            in_e = in_nb;
        }
        // epilogue: O (fp32, tensor memory) -> bf16 -> shared (over the Q tile) -> TMA store
        if (ok) ok = mbar_wait(bar(BAR_OFULL), 0, ctl, W + 10);
        if (ok && args.nsplit > 1) {
            // partial O of this CTA's blocks, fp32, straight from tensor memory to the workspace
            tc_fence_after();
            constexpr int kColsPerGroup = DH / 2;
            const int c0 = group * kColsPerGroup;
            float *dst = args.part + ((((long long)isplit * gridDim.z + b) * args.H + h) * args.S + t) * DH + c0;
#pragma unroll
            for (int g = 0; g < kColsPerGroup / 16; ++g) {
                uint32_t o[16];
                tmem_ld16_sync(lane_base + kColO + c0 + g * 16, o);
                if (in_range) {
#pragma unroll
                    for (int v = 0; v < 4; ++v)
                        *reinterpret_cast<float4 *>(dst + g * 16 + v * 4) =
                            make_float4(__uint_as_float(o[4 * v]), __uint_as_float(o[4 * v + 1]),
                                        __uint_as_float(o[4 * v + 2]), __uint_as_float(o[4 * v + 3]));
                }
            }
            tc_fence_before();
        } else if (ok) {
            tc_fence_after();
            constexpr int kColsPerGroup = DH / 2;  // 64, 48 or 32 columns per thread
            const int c0 = group * kColsPerGroup;
#pragma unroll
            for (int g = 0; g < kColsPerGroup / 16; ++g) {
                uint32_t o[16];
                tmem_ld16_sync(lane_base + kColO + c0 + g * 16, o);
#pragma unroll
                for (int v = 0; v < 2; ++v) {
                    const int col = c0 + g * 16 + v * 8;  // first of 8 columns -> one 16-byte chunk
                    const uint32_t dst = sQ + (col >> 6) * (kBT * 128) + sw128_offset(row, (col & 63) >> 3);
                    st_shared_v4(dst, pack_bf16(__uint_as_float(o[8 * v + 0]), __uint_as_float(o[8 * v + 1])),
                                 pack_bf16(__uint_as_float(o[8 * v + 2]), __uint_as_float(o[8 * v + 3])),
                                 pack_bf16(__uint_as_float(o[8 * v + 4]), __uint_as_float(o[8 * v + 5])),
                                 pack_bf16(__uint_as_float(o[8 * v + 6]), __uint_as_float(o[8 * v + 7])));
                }
            }
            tc_fence_before();
            fence_async_smem();
        }
        named_bar_sync(1, 2 * kGroupThreads);
        if (ok && args.nsplit == 1 && warp == 4 && lane == 0 && !*abort_flag) {
            for (int c = 0; c < L::kChunks; ++c) tma_store_4d(&tmO, sQ + c * (kBT * 128), c * 64, t0, h, b);
            tma_store_commit();
            tma_store_wait_all();
        }
    }

    // ---------------------------------------------------------------------- teardown
    __syncwarp();
    if (*abort_flag) {
        // a wait ran out somewhere in this CTA: give copies and MMAs still in flight time to land
        // before shared and tensor memory are released
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

// O = bf16(sum of the partial O of the splits, in split order); 4 elements per thread.
struct OReduceArgs {
    const float *part;
    long long plane;  // B*H*S*DH
    __nv_bfloat16 *O;
    long long s_b, s_h, s_s;
    int nsplit, H, S, DH;
};
__global__ void __launch_bounds__(256) o_reduce_kernel(const OReduceArgs a) {
    const long long n4 = a.plane / 4;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n4;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long el = idx * 4;
        float4 acc = *reinterpret_cast<const float4 *>(a.part + el);
        for (int s = 1; s < a.nsplit; ++s) {
            const float4 v = *reinterpret_cast<const float4 *>(a.part + (long long)s * a.plane + el);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        const int c = (int)(el % a.DH);
        const long long r1 = el / a.DH;
        const int t = (int)(r1 % a.S);
        const long long r2 = r1 / a.S;
        const int h = (int)(r2 % a.H);
        const long long b = r2 / a.H;
        *reinterpret_cast<uint2 *>(a.O + b * a.s_b + h * a.s_h + t * a.s_s + c) =
            make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
    }
}

struct FwdPlan {
    int nsplit, blocks_per_split;
};
// With fewer token tiles than about half the SMs (decode-shaped calls) the blocks of the intermediate
// dimension are spread over several CTAs per tile so that the weights stream in at full machine rate.
FwdPlan fwd_plan(const flashmhf_dims &d, int num_sms) {
    const long long tiles = (long long)((d.S + kBT - 1) / kBT) * d.H * d.B;
    const int nblk = d.E * d.De / kBI;
    int ns = 1;
    if (tiles < num_sms / 2) ns = (int)((num_sms + tiles - 1) / tiles);
    if (ns > nblk) ns = nblk;
    FwdPlan p;
    p.blocks_per_split = (nblk + ns - 1) / ns;
    p.nsplit = (nblk + p.blocks_per_split - 1) / p.blocks_per_split;  // no empty split
    return p;
}

template <int DH>
int launch_fwd(const flashmhf_fwd_params &p, cudaStream_t st, int *n_launch) {
    using L = FwdSmem<DH>;
    CUtensorMap tmQ, tmK, tmU, tmV, tmO;
    int rc;
    if ((rc = encode_act_map(&tmQ, p.Q, p.d, kBT)) != 0) return rc;
    if ((rc = encode_weight_map(&tmK, p.K, p.d, kBI)) != 0) return rc;
    if ((rc = encode_weight_map(&tmU, p.U, p.d, kBI)) != 0) return rc;
    if ((rc = encode_weight_map(&tmV, p.V, p.d, kBI)) != 0) return rc;
    if ((rc = encode_act_map(&tmO, p.O, p.d, kBT)) != 0) return rc;
    const DeviceCtl *dc = device_ctl();
    if (!dc) return FLASHMHF_ERR_CUDA;
    {  // the attribute is per device and per kernel: set once for each pair
        static std::atomic<bool> done[64];
        if (!done[dc->device].load(std::memory_order_acquire)) {
            cudaError_t e = cudaFuncSetAttribute(fwd_kernel<DH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::kTotal);
            if (e != cudaSuccess) { set_cuda_error(e, "cudaFuncSetAttribute(fwd_kernel)"); return FLASHMHF_ERR_CUDA; }
            done[dc->device].store(true, std::memory_order_release);
        }
    }
    const FwdPlan pl = fwd_plan(p.d, dc->num_sms);
    if (pl.nsplit > 1) {
        if (!p.workspace || p.workspace_bytes < tc_forward_workspace_bytes(p.d) ||
            (reinterpret_cast<uintptr_t>(p.workspace) & 255u))
            return FLASHMHF_ERR_WORKSPACE;
        if (p.O.stride[2] % 4 != 0 || p.O.stride[1] % 4 != 0 || p.O.stride[0] % 4 != 0) return FLASHMHF_ERR_BAD_STRIDE;
    }
    FwdArgs a{static_cast<const float *>(p.R.ptr), p.R.stride[0], p.R.stride[1], p.R.stride[2],
              p.d.S, p.d.E, p.d.De, p.d.H / p.d.Hkuv, pl.nsplit, pl.blocks_per_split,
              static_cast<float *>(p.workspace), p.d.H, 0.5f * p.scale.head_scaling,
              p.scale.head_scaling * p.scale.up_scaling * p.scale.final_scaling, wait_args(dc)};
    dim3 grid(((p.d.S + kBT - 1) / kBT) * pl.nsplit, p.d.H, p.d.B);
    prof_mark(st, kMarkStart);
    fwd_kernel<DH><<<grid, kThreads, L::kTotal, st>>>(tmQ, tmK, tmU, tmV, tmO, a);
    prof_mark(st, kMarkFwd);
    *n_launch += 1;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_cuda_error(e, "fwd_kernel launch"); return FLASHMHF_ERR_CUDA; }
    if (pl.nsplit > 1) {
        const long long plane = (long long)p.d.B * p.d.H * p.d.S * DH;
        OReduceArgs ra{static_cast<const float *>(p.workspace), plane, static_cast<__nv_bfloat16 *>(p.O.ptr),
                       p.O.stride[0], p.O.stride[1], p.O.stride[2], pl.nsplit, p.d.H, p.d.S, DH};
        const long long n4 = plane / 4;
        const long long cap = (long long)dc->num_sms * 4;
        const int blocks = (int)((n4 + 255) / 256 < cap ? (n4 + 255) / 256 : cap);
        o_reduce_kernel<<<blocks, 256, 0, st>>>(ra);
        prof_mark(st, kMarkFwdReduce);
        *n_launch += 1;
        if ((e = cudaGetLastError()) != cudaSuccess) { set_cuda_error(e, "o_reduce_kernel launch"); return FLASHMHF_ERR_CUDA; }
    }
    return FLASHMHF_OK;
}

}  // namespace

size_t tc_forward_workspace_bytes(const flashmhf_dims &d) {
    const DeviceCtl *dc = device_ctl();
    const FwdPlan pl = fwd_plan(d, dc ? dc->num_sms : 148);
    if (pl.nsplit <= 1) return 0;
    return (size_t)pl.nsplit * (size_t)d.B * d.H * d.S * d.Dh * sizeof(float);
}

int tc_forward(const flashmhf_fwd_params &p, cudaStream_t st, int *n_launch) {
    switch (p.d.Dh) {
        case 64: return launch_fwd<64>(p, st, n_launch);
        case 96: return launch_fwd<96>(p, st, n_launch);
        case 128: return launch_fwd<128>(p, st, n_launch);
        default: return FLASHMHF_ERR_BAD_SHAPE;
    }
}

}  // namespace fmhf
