// Forward kernel, bf16, sm_100a:  O = sum_e R_e * ((SiLU(Q K_e^T) * (Q U_e^T)) V_e).
//
// One CTA owns one tile of 128 token rows of one (batch, head).  Its Q tile is loaded once; the
// weights of the head stream through shared-memory rings, 64 intermediate rows (one "block": 64
// rows of K_e, U_e and V_e) at a time.  Per block the tensor core computes
//     S = Q [K_blk; U_blk]^T      (128 x 128, one MMA chain, fp32 in tensor memory: M | N)
// the activation warps read S, form A = bf16(SiLU(M) * N * R_e) in registers and write it back into
// tensor memory (two bf16 per column), and the tensor core accumulates, with A read from tensor memory
// and V from shared memory,
//     O += A V_blk                (128 x d_h, fp32 in tensor memory, over all blocks of all e)
// so the [T, E*d_e] intermediate never leaves the SM and A never touches shared memory.
//
// Pipeline.  The hand-off from an MMA to the warps that consume its result costs several hundred
// cycles (commit -> mbarrier -> wake-up) and the tensor pipe accepts MMAs only a few ahead of their
// execution, so nothing on the S path waits for anything on the O path:
//   * Q is copied once from shared into tensor memory and the S chain reads it from there: an MMA with both
//     operands in shared memory uses the whole shared-memory bandwidth of the SM (measured: 128x128x16 takes
//     64.5 clk = 8 KB at 128 B/clk), which the weight tiles arriving by TMA need as well.
//   * S has two buffers.  A thread's first step on a block is to load its part of M and N into registers,
//     after which the buffer is free again -- S of block j+2 may be issued while block j is still being activated.
//   * A has slots of its own (32 columns each), so the O update of a block may lag its activation without
//     holding an S buffer.
//   * The two MMA chains are issued by different threads (S by two threads, one per S buffer, so that each
//     sees every phase of the barriers of its buffer; O by a third).
//
// Warp roles: warp 0 TMA producer, warps 1-2 MMA issuers for S (even / odd blocks; warp 1 owns tensor
// memory), warp 3 MMA issuer for O, then the activation warps (warp % 4 = TMEM lane quarter = 32 token rows).
//
// Tensor memory (512 columns): O at [0, d_h), Q (bf16) at [128, 192), A slots at [192, 256), S buffers at
// [256, 384), [384, 512).
#include <atomic>

#include "kernels.h"
#include "tc_common.cuh"
#include <utility>
#include "tensormap.cuh"

namespace fmhf {
namespace {

constexpr int kBT = 128;  // token rows per tile
constexpr int kBI = 64;   // intermediate rows per block
// Shared-memory stages of the [K;U] ring and of the V ring (two Q tiles take the rest).  The [K;U] ring must have an
// EVEN number of stages: its "full" barriers are waited on by the two S issuers, which own alternate blocks, and a
// barrier's phase is tracked with one parity bit, so each stage must always be waited on by the same issuer (with an
// odd ring an issuer would meet a stage only every other time it fills and could take an old phase for the new one).
constexpr int kKURing = 4, kVRing = 2;
static_assert(kKURing % 2 == 0, "each [K;U] stage must belong to one S issuer");
// Activation teams of eight warps (warp % 4 = lane quarter, next bit = which 32 of a block's 64 columns).  With two
// teams, team t owns the blocks j = t (mod 2) and with them S buffer t and A slot t; the two teams are then in
// different phases of their loop (wait, load, arithmetic, store), which keeps the arithmetic pipes busy.
// One team at d_h = 128, where the kernel is paced by the arrival of the weight tiles from L2 (48 KB per block at
// about 50 B/clk per SM) and by the tensor pipe; two teams at d_h = 64 and 96, where it is paced by the activation.
constexpr int kTeamThreads = 256;
__host__ __device__ constexpr int teams_for(int dh) { return dh == 128 ? 1 : 2; }
__host__ __device__ constexpr int threads_for(int dh) { return 128 + teams_for(dh) * kTeamThreads; }
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColO = 0, kColQ = 128, kColA0 = 192, kColAStride = 32, kColS0 = 256, kColSStride = 128;

template <int DH>
struct FwdSmem {
    static constexpr int kChunks = (DH + 63) / 64;              // 64-column SW128 chunks per row of d_h
    static constexpr uint32_t kQBytes = kChunks * kBT * 128;    // one Q tile (also the O staging tile of its work item)
    static constexpr uint32_t kWChunk = kBI * 128;              // one 64-row x 64-col weight chunk
    static constexpr uint32_t kKUStage = 2 * kChunks * kWChunk; // per chunk: K rows then U rows = one 128-row K-major tile
    static constexpr uint32_t kVStage = kChunks * kWChunk;
    // offsets from the 1024-aligned base
    static constexpr uint32_t kOffQ = 0;                        // two Q tiles: work items alternate between them
    static constexpr uint32_t kOffKU = kOffQ + 2 * kQBytes;
    static constexpr uint32_t kOffV = kOffKU + kKURing * kKUStage;
    static constexpr uint32_t kOffBar = kOffV + kVRing * kVStage;
    static constexpr uint32_t kTotal = kOffBar + 320 + 1024;  // + barriers/control + alignment slack
};

// barrier slots (8 bytes each) inside the control area
// QFULL[q]: Q tile q has landed; QFREE[q]: the O tile staged over it has been read by its TMA store;
// SFULL[b]: S computed into buffer b; SEMPTY[b]: every warp of the team working on it has its part in registers;
// AFULL[s]: A written to slot s; AFREE[s]: the O update that read slot s is done; QT: Q copied to tensor memory;
// OFULL: the last O update of a work item is done; OFREE: its accumulator has been read out.
// A CTA walks several work items (token tiles); blocks are counted through all of them (g), buffer and slot of a block
// are g % 2, Q tile and per-item barriers alternate with the item count, so every barrier has one fixed set of
// waiters that observes each of its phases and a one-bit phase parity is enough.
enum { BAR_QFULL = 0, BAR_QFREE = 2, BAR_KUFULL = 4, BAR_KUEMPTY = 8, BAR_VFULL = 12, BAR_VEMPTY = 16, BAR_SFULL = 20,  // rings: up to 4 stages
       BAR_SEMPTY = 22, BAR_AFULL = 24, BAR_AFREE = 26, BAR_OFULL = 28, BAR_OFREE = 29, BAR_QT = 30, BAR_COUNT = 31 };

struct FwdArgs {
    const float *R;
    long long r_sb, r_sh, r_ss;
    int S, E, De, G;
    // Split of the intermediate dimension over CTAs (short token counts, e.g. decode): a work item is (token tile,
    // split) and covers blocks [isplit * blocks_per_split, ...) of the tile; it writes an fp32 partial O.
    int nsplit, blocks_per_split;
    float *part;           // [nsplit][B][H][S][DH] fp32, used when nsplit > 1
    int H, B;
    int tiles_per_seq, n_items;   // work items = tiles_per_seq * H * B * nsplit, dealt round-robin to the CTAs
    float half_s0;  // 0.5 * head_scaling: tanh argument scale, sigmoid(s0 m) = 0.5 + 0.5 tanh(0.5 s0 m)
    float c;        // head_scaling * up_scaling * final_scaling, folded into the routing weight
    // Chained call: launched with programmatic stream serialization.  The CTA may start, and stream weight tiles,
    // while the kernel before it on the stream still runs; Q and R are read, and anything written, only after
    // griddep_wait().
    int chained;
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

// A work item: which token tile of which (batch, head), which blocks of the intermediate dimension.
struct FwdItem {
    int t0, h, b, isplit, j0, nblk;
};
__device__ __forceinline__ FwdItem fwd_item(const FwdArgs &a, int item, int nblk_total) {
    FwdItem w;
    w.isplit = item % a.nsplit;
    int t = item / a.nsplit;
    w.t0 = (t % a.tiles_per_seq) * kBT;
    t /= a.tiles_per_seq;
    w.h = t % a.H;
    w.b = t / a.H;
    w.j0 = w.isplit * a.blocks_per_split;
    w.nblk = min(nblk_total - w.j0, a.blocks_per_split);
    return w;
}

template <int DH>
__global__ void __launch_bounds__(threads_for(DH), 1)
fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
           const __grid_constant__ CUtensorMap tmU, const __grid_constant__ CUtensorMap tmV,
           const __grid_constant__ CUtensorMap tmO, const FwdArgs args) {
    using L = FwdSmem<DH>;
    constexpr int kTeams = teams_for(DH);
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *gbase = smem_raw + (base - raw);
    const uint32_t sQ = base + L::kOffQ, sKU = base + L::kOffKU, sV = base + L::kOffV, sBar = base + L::kOffBar;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(gbase + L::kOffBar + BAR_COUNT * 8);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(gbase + L::kOffBar + BAR_COUNT * 8 + 4);
    auto bar = [&](int i) { return sBar + 8u * i; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int blocks_per_e = args.De / kBI, nblk_total = args.E * blocks_per_e;
    const WaitCtl ctl{abort_flag, args.wait};
    constexpr int W = kKernelFwd * 100;

    if (threadIdx.x == 0) {
        *abort_flag = launch_aborted(args.wait);  // a CTA of this launch gave up: drain fast
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar(BAR_QFULL + i), 1);
            mbar_init(bar(BAR_QFREE + i), 1);
            mbar_init(bar(BAR_SFULL + i), 1);
            mbar_init(bar(BAR_SEMPTY + i), arrivals_of(kTeamThreads));
            mbar_init(bar(BAR_AFULL + i), arrivals_of(kTeamThreads));
            mbar_init(bar(BAR_AFREE + i), 1);
        }
        for (int i = 0; i < kKURing; ++i) {
            mbar_init(bar(BAR_KUFULL + i), 1);
            mbar_init(bar(BAR_KUEMPTY + i), 1);
        }
        for (int i = 0; i < kVRing; ++i) {
            mbar_init(bar(BAR_VFULL + i), 1);
            mbar_init(bar(BAR_VEMPTY + i), 1);
        }
        mbar_init(bar(BAR_OFULL), 1);
        mbar_init(bar(BAR_OFREE), arrivals_of(kTeamThreads));
        mbar_init(bar(BAR_QT), arrivals_of(kTeamThreads));
        fence_mbar_init();
    }
    if (warp == 1) tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const bool dead = *abort_flag != 0;
    if (args.chained) griddep_launch_dependents();   // every CTA of this launch is running: the next call may start

    if (dead) {
        // nothing: fall through to the teardown
    } else if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            tma_prefetch_desc(&tmQ);
            tma_prefetch_desc(&tmK);
            tma_prefetch_desc(&tmU);
            tma_prefetch_desc(&tmV);
            RingPos<kKURing> pk;
            RingPos<kVRing> pv;
            bool ok = true;
            int n = 0;  // work items of this CTA so far
            for (int item = blockIdx.x; ok && item < args.n_items; item += gridDim.x, ++n) {
                const FwdItem w = fwd_item(args, item, nblk_total);
                const int hk = w.h / args.G, q = n & 1;
                // the Q tile of item n - 2 doubled as its O staging tile: wait until its store has read it
                if (n >= 2 && !mbar_wait(bar(BAR_QFREE + q), ((n >> 1) - 1) & 1, ctl, W + 12)) break;
                // (the first Q of a chained call is asked for by the activation warps, once the kernel before this one has
                // completed: this thread touches only the weights and never waits for that)
                if (!(args.chained && n == 0)) {
                    mbar_arrive_expect_tx(bar(BAR_QFULL + q), L::kQBytes);
                    for (int c = 0; c < L::kChunks; ++c)
                        tma_load_4d(sQ + q * L::kQBytes + c * (kBT * 128), &tmQ, bar(BAR_QFULL + q), c * 64, w.t0, w.h, w.b);
                }
                // [K;U] of block j, then V of block j-2: V is consumed about two blocks later than K and U of
                // the same block, so with this lag the producer never waits on the V ring while a [K;U]
                // stage is free.
                for (int j = 0; j < w.nblk + 2; ++j) {
                    if (j < w.nblk) {
                        if (!mbar_wait(bar(BAR_KUEMPTY + pk.slot), pk.lap ^ 1, ctl, W + 1)) { ok = false; break; }
                        const uint32_t fku = bar(BAR_KUFULL + pk.slot), dku = sKU + pk.slot * L::kKUStage;
                        mbar_arrive_expect_tx(fku, L::kKUStage);
#pragma unroll
                        for (int c = 0; c < L::kChunks; ++c) {
                            tma_load_3d(dku + c * 2 * L::kWChunk, &tmK, fku, c * 64, (w.j0 + j) * kBI, hk);
                            tma_load_3d(dku + c * 2 * L::kWChunk + L::kWChunk, &tmU, fku, c * 64, (w.j0 + j) * kBI, hk);
                        }
                        pk.advance(1);
                    }
                    if (j >= 2) {
                        if (!mbar_wait(bar(BAR_VEMPTY + pv.slot), pv.lap ^ 1, ctl, W + 2)) { ok = false; break; }
                        const uint32_t fv = bar(BAR_VFULL + pv.slot), dv = sV + pv.slot * L::kVStage;
                        mbar_arrive_expect_tx(fv, L::kVStage);
#pragma unroll
                        for (int c = 0; c < L::kChunks; ++c)
                            tma_load_3d(dv + c * L::kWChunk, &tmV, fv, c * 64, (w.j0 + j - 2) * kBI, hk);
                        pv.advance(1);
                    }
                }
            }
        }
    } else if (warp == 1 || warp == 2) {
        // ------------------------------------------------------------------ MMA issuers for S = Q [K;U]^T
        // Two threads (warp 1: even blocks into S buffer 0, warp 2: odd blocks into buffer 1; blocks counted through all
        // work items of the CTA): while one is between batches -- barrier polls, commits -- the other keeps the tensor
        // pipe fed.  Q is read from tensor memory.  One thread issues a chain, so its instruction stream is kept
        // minimal: descriptors are built once and advanced by adding constants (the address field counts 16-byte units).
        if (lane == 0) {
            constexpr uint32_t idesc1 = umma_idesc(128, 2 * kBI, false, false);
            const uint64_t dKU0 = desc_kmajor(sKU);
            constexpr uint64_t kKUStep = L::kKUStage >> 4;
            const int sb = warp - 1;
            const uint32_t tS = tmem + kColS0 + sb * kColSStride, tQ = tmem + kColQ;
            bool ok = true;
            int g0 = 0, n = 0;   // blocks before this work item; work items so far
            for (int item = blockIdx.x; ok && item < args.n_items; item += gridDim.x, ++n) {
                const FwdItem w = fwd_item(args, item, nblk_total);
                if (!mbar_wait(bar(BAR_QT), n & 1, ctl, W + 3)) break;   // this item's Q is in tensor memory
                for (int j = (g0 + sb) & 1; j < w.nblk; j += 2) {
                    const int g = g0 + j;                                 // g % 2 == sb
                    const int slot = g % kKURing;
                    if (!mbar_wait(bar(BAR_KUFULL + slot), (g / kKURing) & 1, ctl, W + 4)) { ok = false; break; }
                    // the buffer's previous block (g - 2) is in the activation warps' registers
                    if (g >= 2 && !mbar_wait(bar(BAR_SEMPTY + sb), ((g >> 1) - 1) & 1, ctl, W + 5)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t dku = dKU0 + slot * kKUStep;
#pragma unroll
                    for (int k = 0; k < DH / 16; ++k) {
                        const int c = k >> 2, kk = k & 3;
                        umma_ts(tS, tQ + k * 8, dku + ((c * 2 * L::kWChunk + kk * 32) >> 4), idesc1, k > 0 ? 1u : 0u);
                    }
                    umma_commit(bar(BAR_KUEMPTY + slot));
                    umma_commit(bar(BAR_SFULL + sb));
                }
                g0 += w.nblk;
            }
        }
    } else if (warp == 3) {
        // ------------------------------------------------------------------ MMA issuer 2: O += A V
        // A comes from tensor memory (slot g % 2), V from shared memory as an MN-major operand.
        if (lane == 0) {
            constexpr uint32_t idesc2 = umma_idesc(128, DH, false, true);
            const uint64_t dV0 = desc_mnmajor(sV, L::kWChunk);
            constexpr uint64_t kVStep = L::kVStage >> 4;
            bool ok = true;
            int g0 = 0, n = 0;
            for (int item = blockIdx.x; ok && item < args.n_items; item += gridDim.x, ++n) {
                const FwdItem w = fwd_item(args, item, nblk_total);
                // the accumulator of the previous work item has been read out
                if (n >= 1 && !mbar_wait(bar(BAR_OFREE), (n - 1) & 1, ctl, W + 13)) break;
                for (int j = 0; j < w.nblk; ++j) {
                    const int g = g0 + j, slot = g & 1, vs = g % kVRing;
                    if (!mbar_wait(bar(BAR_VFULL + vs), (g / kVRing) & 1, ctl, W + 6)) { ok = false; break; }
                    if (!mbar_wait(bar(BAR_AFULL + slot), (g >> 1) & 1, ctl, W + 7)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t dv = dV0 + vs * kVStep;
                    const uint32_t tA = tmem + kColA0 + slot * kColAStride;
#pragma unroll
                    for (int k = 0; k < kBI / 16; ++k)
                        umma_ts(tmem + kColO, tA + k * 8, dv + k * 128, idesc2, (j > 0 || k > 0) ? 1u : 0u);
                    umma_commit(bar(BAR_VEMPTY + vs));
                    umma_commit(bar(BAR_AFREE + slot));
                }
                if (ok) umma_commit(bar(BAR_OFULL));
                g0 += w.nblk;
            }
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------------ activation + epilogue
        const int quarter = warp & 3, team = (warp - 4) >> 3, group = ((warp - 4) >> 2) & 1;  // group = column half
        const int row = quarter * 32 + lane;
        const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
        const f32x2 half_s0 = f2_pack(args.half_s0, args.half_s0);
        bool ok = true;
        int g0 = 0, n = 0;   // blocks before this work item; work items so far
        if (args.chained) {
            griddep_wait();   // these warps read R and write O
            if (warp == 4 && lane == 0 && blockIdx.x < args.n_items) {   // the first item's Q (q.v. the producer)
                const FwdItem w = fwd_item(args, blockIdx.x, nblk_total);
                mbar_arrive_expect_tx(bar(BAR_QFULL), L::kQBytes);
                for (int c = 0; c < L::kChunks; ++c)
                    tma_load_4d(sQ + c * (kBT * 128), &tmQ, bar(BAR_QFULL), c * 64, w.t0, w.h, w.b);
            }
            __syncwarp();
        }
        // Copy of a work item's Q tile from shared into tensor memory, by team 0 (thread = token row; its lower four warps
        // copy columns [0, 64) of d_h, the upper four [64, 128)).  Done as soon as the previous item's last S has been
        // read, i.e. before that item's epilogue, so that the first S of the new item is computed under the epilogue.
        auto copy_q = [&](int nn) -> bool {
            if (!mbar_wait(bar(BAR_QFULL + (nn & 1)), (nn >> 1) & 1, ctl, W + 11)) return false;
            if (group * 64 < DH) {
                uint32_t qv[32];
                const uint8_t *src = gbase + L::kOffQ + (nn & 1) * L::kQBytes + group * (kBT * 128);
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint4 v = *reinterpret_cast<const uint4 *>(src + sw128_offset(row, c));
                    qv[4 * c] = v.x; qv[4 * c + 1] = v.y; qv[4 * c + 2] = v.z; qv[4 * c + 3] = v.w;
                }
                tmem_st32(lane_base + kColQ + group * 32, qv);
                tmem_st_wait();
            }
            tc_fence_before();
            warp_arrive(bar(BAR_QT));
            return true;
        };
        if (team == 0 && blockIdx.x < args.n_items) ok = copy_q(0);
        for (int item = blockIdx.x; ok && item < args.n_items; item += gridDim.x, ++n) {
            const FwdItem w = fwd_item(args, item, nblk_total);
            const int t = w.t0 + row;
            const bool in_range = t < args.S;
            const float *rrow = args.R + (long long)w.b * args.r_sb + (long long)w.h * args.r_sh + (long long)t * args.r_ss;
            // this team's first block of the item, its sub-network and position inside it; routing weight fetched one ahead
            const int jfirst = kTeams == 1 ? 0 : ((g0 + team) & 1);
            int e = (w.j0 + jfirst) / blocks_per_e, in_e = (w.j0 + jfirst) - e * blocks_per_e;
            float r_cur = (in_range && e < args.E) ? __ldg(rrow + e) : 0.f;
            float r_next = (in_range && e + 1 < args.E) ? __ldg(rrow + e + 1) : 0.f;
            for (int j = jfirst; j < w.nblk; j += kTeams) {
                const int g = g0 + j, sb = g & 1;   // S buffer and A slot of this block
                const float hr = 0.5f * args.c * r_cur;
                const f32x2 half_r = f2_pack(hr, hr);
                if (!mbar_wait(bar(BAR_SFULL + sb), (g >> 1) & 1, ctl, W + 8)) { ok = false; break; }
                tc_fence_after();
                const uint32_t ts = lane_base + kColS0 + sb * kColSStride + group * 32;
                uint32_t m[32], nn[32], a[16];  // this thread's 32 columns of M and of N; 32 bf16 of A
                tmem_ld32x2_sync(ts, ts + kBI, m, nn);
                tc_fence_before();
                warp_arrive(bar(BAR_SEMPTY + sb));  // S is in registers: the buffer may take block g + 2
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    a[i] = fwd_act_pair(f2_pack_bits(m[2 * i], m[2 * i + 1]), f2_pack_bits(nn[2 * i], nn[2 * i + 1]), half_r,
                                        half_s0);
                // the slot's previous block (g - 2) has been consumed by its O update
                if (g >= 2 && !mbar_wait(bar(BAR_AFREE + sb), ((g >> 1) - 1) & 1, ctl, W + 9)) { ok = false; break; }
                tc_fence_after();
                tmem_st16(lane_base + kColA0 + sb * kColAStride + group * 16, a);
                tmem_st_wait();
                tc_fence_before();
                warp_arrive(bar(BAR_AFULL + sb));
#pragma unroll
                for (int k = 0; k < kTeams; ++k)
                    if (++in_e == blocks_per_e) {
                        in_e = 0;
                        ++e;
                        r_cur = r_next;
                        r_next = (in_range && e + 1 < args.E) ? __ldg(rrow + e + 1) : 0.f;
                    }
            }
            g0 += w.nblk;
            if (!ok || team != 0) continue;   // the rest of the item is team 0's
            // every S of this item has been read: the next item's Q may replace it in tensor memory
            if (item + (int)gridDim.x < args.n_items && !copy_q(n + 1)) { ok = false; break; }
            // epilogue: O (fp32, tensor memory) -> bf16 -> shared (over this item's Q tile) -> TMA store
            if (!mbar_wait(bar(BAR_OFULL), n & 1, ctl, W + 10)) { ok = false; break; }
            tc_fence_after();
            constexpr int kColsPerGroup = DH / 2;  // 64, 48 or 32 columns per thread
            const int c0 = group * kColsPerGroup;
            const uint32_t sO = sQ + (n & 1) * L::kQBytes;
            if (args.nsplit > 1) {
                // partial O of this item's blocks, fp32, straight from tensor memory to the workspace
                float *dst = args.part + ((((long long)w.isplit * args.B + w.b) * args.H + w.h) * args.S + t) * DH + c0;
#pragma unroll
                for (int gg = 0; gg < kColsPerGroup / 16; ++gg) {
                    uint32_t o[16];
                    tmem_ld16_sync(lane_base + kColO + c0 + gg * 16, o);
                    if (in_range) {
#pragma unroll
                        for (int v = 0; v < 4; ++v)
                            *reinterpret_cast<float4 *>(dst + gg * 16 + v * 4) =
                                make_float4(__uint_as_float(o[4 * v]), __uint_as_float(o[4 * v + 1]),
                                            __uint_as_float(o[4 * v + 2]), __uint_as_float(o[4 * v + 3]));
                    }
                }
                tc_fence_before();
                warp_arrive(bar(BAR_OFREE));
            } else {
#pragma unroll
                for (int gg = 0; gg < kColsPerGroup / 16; ++gg) {
                    uint32_t o[16];
                    tmem_ld16_sync(lane_base + kColO + c0 + gg * 16, o);
#pragma unroll
                    for (int v = 0; v < 2; ++v) {
                        const int col = c0 + gg * 16 + v * 8;  // first of 8 columns -> one 16-byte chunk
                        const uint32_t dst = sO + (col >> 6) * (kBT * 128) + sw128_offset(row, (col & 63) >> 3);
                        st_shared_v4(dst, pack_bf16(__uint_as_float(o[8 * v + 0]), __uint_as_float(o[8 * v + 1])),
                                     pack_bf16(__uint_as_float(o[8 * v + 2]), __uint_as_float(o[8 * v + 3])),
                                     pack_bf16(__uint_as_float(o[8 * v + 4]), __uint_as_float(o[8 * v + 5])),
                                     pack_bf16(__uint_as_float(o[8 * v + 6]), __uint_as_float(o[8 * v + 7])));
                    }
                }
                tc_fence_before();
                warp_arrive(bar(BAR_OFREE));   // the accumulator is in registers / shared memory: the next item may overwrite it
                fence_async_smem();
                named_bar_sync(1, kTeamThreads);
                if (warp == 4 && lane == 0) {
                    for (int c = 0; c < L::kChunks; ++c) tma_store_4d(&tmO, sO + c * (kBT * 128), c * 64, w.t0, w.h, w.b);
                    tma_store_commit();
                    tma_store_wait_read();          // the tile has been read: it may take the Q of the item after next
                    mbar_arrive(bar(BAR_QFREE + (n & 1)));
                }
            }
        }
        if (warp == 4 && lane == 0) tma_store_wait_all();
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
    int chained;   // launched with programmatic stream serialization, between two chained forward kernels
};
// 128 threads and few registers: its CTAs fit beside the forward kernel's on an SM, so a chained launch is resident (and
// has let the next forward launch in turn) long before the forward kernel it waits for ends.
__global__ void __maxnreg__(48) o_reduce_kernel(const OReduceArgs a) {
    if (a.chained) {
        griddep_launch_dependents();
        griddep_wait();
    }
    // Every thread takes two 16-byte pieces of O at a time and has the loads of three splits of both in flight at once
    // (the partial sums come from L2 while the next call's weights stream in from HBM: latency is what this kernel is
    // made of); the splits are added in index order.  48 registers: 128 threads of it fit beside the d_h = 128 forward CTA.
    // (a split call has fewer than SMs / 2 token tiles: every index fits 32 bits)
    const int n4 = (int)(a.plane / 4), stride = (int)(gridDim.x * blockDim.x);
    auto store = [&](int idx, const float4 &acc) {
        const int per_row = a.DH / 4;
        const int r1 = idx / per_row, c = (idx - r1 * per_row) * 4;
        const int r2 = r1 / a.S, t = r1 - r2 * a.S;
        const int b = r2 / a.H, h = r2 - b * a.H;
        *reinterpret_cast<uint2 *>(a.O + (long long)b * a.s_b + (long long)h * a.s_h + (long long)t * a.s_s + c) =
            make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
    };
    const float4 *part4 = reinterpret_cast<const float4 *>(a.part);
    const int plane4 = n4;
    for (int idx = (int)(blockIdx.x * blockDim.x + threadIdx.x); idx < n4; idx += 2 * stride) {
        const bool two = idx + stride < n4;
        const int idx1 = two ? idx + stride : idx;
        float4 acc0 = __ldcg(part4 + idx), acc1 = __ldcg(part4 + idx1);
        for (int s0 = 1; s0 < a.nsplit; s0 += 3) {
            float4 v0[3], v1[3];
#pragma unroll
            for (int k = 0; k < 3; ++k) {
                const float4 *src = part4 + (long long)min(s0 + k, a.nsplit - 1) * plane4;
                v0[k] = __ldcg(src + idx);
                v1[k] = __ldcg(src + idx1);
            }
#pragma unroll
            for (int k = 0; k < 3; ++k) {
                if (s0 + k < a.nsplit) {
                    acc0.x += v0[k].x; acc0.y += v0[k].y; acc0.z += v0[k].z; acc0.w += v0[k].w;
                    acc1.x += v1[k].x; acc1.y += v1[k].y; acc1.z += v1[k].z; acc1.w += v1[k].w;
                }
            }
        }
        store(idx, acc0);
        if (two) store(idx1, acc1);
    }
}

struct FwdPlan {
    int nsplit, blocks_per_split;
};
// With fewer token tiles than about half the SMs (decode-shaped calls) the blocks of the intermediate
// dimension are spread over several CTAs per tile so that the weights stream in at full machine rate.
// All CTAs must run at once: one CTA per SM, so tiles * splits never exceeds the SM count (a second,
// nearly empty wave would double the duration of a call that lasts tens of microseconds).
FwdPlan fwd_plan(const flashmhf_dims &d, int num_sms) {
    const long long tiles = (long long)((d.S + kBT - 1) / kBT) * d.H * d.B;
    const int nblk = d.E * d.De / kBI;
    int ns = 1;
    if (tiles < num_sms / 2) ns = (int)(num_sms / tiles);
    if (ns > nblk) ns = nblk;
    FwdPlan p;
    p.blocks_per_split = (nblk + ns - 1) / ns;
    p.nsplit = (nblk + p.blocks_per_split - 1) / p.blocks_per_split;  // no empty split
    return p;
}

// Launch with programmatic stream serialization: the kernel may start before the one ahead of it on the stream has ended.
template <typename... KArgs, typename... Args>
cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

template <int DH>
int launch_fwd(const flashmhf_fwd_params &p, cudaStream_t st, int *n_launch, bool chained) {
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
    {  // the attributes are per device and per kernel: set once for each pair
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
              static_cast<float *>(p.workspace), p.d.H, p.d.B, 0, 0, 0.5f * p.scale.head_scaling,
              p.scale.head_scaling * p.scale.up_scaling * p.scale.final_scaling, chained ? 1 : 0, wait_args(dc)};
    a.tiles_per_seq = (p.d.S + kBT - 1) / kBT;
    const long long items = (long long)a.tiles_per_seq * p.d.H * p.d.B * pl.nsplit;
    if (items > 0x7fffffffLL) return FLASHMHF_ERR_BAD_SHAPE;
    a.n_items = (int)items;
    // one CTA per SM walks the work items round-robin: the next item's Q load, Q copy and first S overlap this item's epilogue
    // (a split call has one item per CTA: tiles * splits <= SMs)
    const unsigned grid = (unsigned)(items < dc->num_sms ? items : dc->num_sms);
    prof_mark(st, kMarkStart);
    cudaError_t e;
    if (chained) {
        e = launch_chained(fwd_kernel<DH>, dim3(grid), dim3(threads_for(DH)), L::kTotal, st, tmQ, tmK, tmU, tmV, tmO, a);
    } else {
        fwd_kernel<DH><<<grid, threads_for(DH), L::kTotal, st>>>(tmQ, tmK, tmU, tmV, tmO, a);
        e = cudaGetLastError();
    }
    prof_mark(st, kMarkFwd);
    *n_launch += 1;
    if (e != cudaSuccess) { set_cuda_error(e, "fwd_kernel launch"); return FLASHMHF_ERR_CUDA; }
    if (pl.nsplit > 1) {
        const long long plane = (long long)p.d.B * p.d.H * p.d.S * DH;
        OReduceArgs ra{static_cast<const float *>(p.workspace), plane, static_cast<__nv_bfloat16 *>(p.O.ptr),
                       p.O.stride[0], p.O.stride[1], p.O.stride[2], pl.nsplit, p.d.H, p.d.S, DH, chained ? 1 : 0};
        const long long n4 = plane / 4;
        // chained: at most one (small) CTA per SM, so that all of them are resident beside the forward kernel's
        const long long cap = chained ? (long long)dc->num_sms : (long long)dc->num_sms * 8;
        const int blocks = (int)((n4 + 127) / 128 < cap ? (n4 + 127) / 128 : cap);
        if (chained) e = launch_chained(o_reduce_kernel, dim3(blocks), dim3(128), 0, st, ra);
        else o_reduce_kernel<<<blocks, 128, 0, st>>>(ra);
        prof_mark(st, kMarkFwdReduce);
        *n_launch += 1;
        if (!chained) e = cudaGetLastError();
        if (e != cudaSuccess) { set_cuda_error(e, "o_reduce_kernel launch"); return FLASHMHF_ERR_CUDA; }
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

int tc_forward(const flashmhf_fwd_params &p, cudaStream_t st, int *n_launch, bool chained) {
    switch (p.d.Dh) {
        case 64: return launch_fwd<64>(p, st, n_launch, chained);
        case 96: return launch_fwd<96>(p, st, n_launch, chained);
        case 128: return launch_fwd<128>(p, st, n_launch, chained);
        default: return FLASHMHF_ERR_BAD_SHAPE;
    }
}

}  // namespace fmhf
