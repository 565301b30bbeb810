// Forward kernel, bf16, sm_100a:  O = sum_e R_e * ((SiLU(Q K_e^T) * (Q U_e^T)) V_e).
//
// One CTA owns one tile of 128 token rows of one (batch, head).  Its Q tile is loaded once; the
// weights of the head stream through a ring of shared-memory stages, 64 intermediate rows
// (one "block": 64 rows of K_e, U_e and V_e) per stage.  Per block the tensor core computes
//     S = Q [K_blk; U_blk]^T      (128 x 128, one MMA chain, fp32 in tensor memory: M | N)
// the activation warps read S, form A = bf16(SiLU(M) * N * R_e) in registers and write it to a
// shared-memory operand tile, and the tensor core accumulates
//     O += A V_blk                (128 x d_h, fp32 in tensor memory, over all blocks of all e)
// so the [T, E*d_e] intermediate never leaves the SM.  S and A are double-buffered so the MMA of
// block j+1 overlaps the activation of block j.
//
// Warp roles (384 threads): warp 0 TMA producer, warp 1 MMA issuer + tensor-memory owner,
// warps 2-3 idle, warps 4-11 activation/epilogue (warp % 4 = TMEM lane quarter = 32 token rows,
// (warp-4)/4 = which 32 of the block's 64 intermediate columns).
//
// Tensor memory (512 columns): O at [0, d_h), S buffers at [128, 256) and [256, 384).
#include "kernels.h"
#include "tc_common.cuh"
#include "tensormap.cuh"

namespace fmhf {
namespace {

constexpr int kBT = 128;  // token rows per tile
constexpr int kBI = 64;   // intermediate rows per block
constexpr int kStages = 3;
constexpr int kThreads = 384;
constexpr int kActThreads = 256;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColO = 0, kColS0 = 128, kColSStride = 128;

template <int DH>
struct FwdSmem {
    static constexpr int kChunks = (DH + 63) / 64;              // 64-column SW128 chunks per row of d_h
    static constexpr uint32_t kQBytes = kChunks * kBT * 128;    // Q tile (also the O staging tile)
    static constexpr uint32_t kWChunk = kBI * 128;              // one 64-row x 64-col weight chunk
    static constexpr uint32_t kStageBytes = 3 * kChunks * kWChunk;
    static constexpr uint32_t kABytes = kBT * 128;              // A tile: 128 rows x 64 cols
    // offsets from the 1024-aligned base
    static constexpr uint32_t kOffQ = 0;
    static constexpr uint32_t kOffW = kOffQ + kQBytes;
    static constexpr uint32_t kOffA = kOffW + kStages * kStageBytes;
    static constexpr uint32_t kOffBar = kOffA + 2 * kABytes;
    static constexpr uint32_t kTotal = kOffBar + 256 + 1024;  // + barriers/control + alignment slack
    // inside a stage: chunk c of K at c*2*kWChunk, of U right behind it (so [K;U] of one chunk is one
    // 128-row K-major tile), V chunks after all K/U chunks.
    static constexpr uint32_t kOffV = 2 * kChunks * kWChunk;
};

// barrier slots (8 bytes each) inside the control area
enum { BAR_Q = 0, BAR_WFULL = 1, BAR_WEMPTY = 4, BAR_SFULL = 7, BAR_SEMPTY = 9, BAR_AFULL = 11, BAR_AEMPTY = 13,
       BAR_OFULL = 15, BAR_COUNT = 16 };

struct FwdArgs {
    const float *R;
    long long r_sb, r_sh, r_ss;
    int S, E, De, G;
    int *status;
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
    const uint32_t sQ = base + L::kOffQ, sW = base + L::kOffW, sA = base + L::kOffA, sBar = base + L::kOffBar;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(gbase + L::kOffBar + BAR_COUNT * 8);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(gbase + L::kOffBar + BAR_COUNT * 8 + 4);
    auto bar = [&](int i) { return sBar + 8u * i; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = blockIdx.x * kBT, h = blockIdx.y, b = blockIdx.z, hk = h / args.G;
    const int blocks_per_e = args.De / kBI;
    const int nblk = args.E * blocks_per_e;
    const WaitCtl ctl{abort_flag, args.status};
    constexpr int W = kKernelFwd * 100;

    if (threadIdx.x == 0) {
        *abort_flag = (*reinterpret_cast<volatile int *>(args.status) != 0);  // an earlier CTA gave up: drain fast
        mbar_init(bar(BAR_Q), 1);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar(BAR_WFULL + s), 1);
            mbar_init(bar(BAR_WEMPTY + s), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar(BAR_SFULL + i), 1);
            mbar_init(bar(BAR_SEMPTY + i), kActThreads);
            mbar_init(bar(BAR_AFULL + i), kActThreads);
            mbar_init(bar(BAR_AEMPTY + i), 1);
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
            for (int j = 0; j < nblk; ++j) {
                const int s = j % kStages, n = j / kStages;
                if (!mbar_wait(bar(BAR_WEMPTY + s), (n & 1) ^ 1, ctl, W + 1)) break;
                const uint32_t st = sW + s * L::kStageBytes;
                mbar_arrive_expect_tx(bar(BAR_WFULL + s), L::kStageBytes);
                const int row = j * kBI;
                for (int c = 0; c < L::kChunks; ++c) {
                    tma_load_3d(st + c * 2 * L::kWChunk, &tmK, bar(BAR_WFULL + s), c * 64, row, hk);
                    tma_load_3d(st + c * 2 * L::kWChunk + L::kWChunk, &tmU, bar(BAR_WFULL + s), c * 64, row, hk);
                }
                for (int c = 0; c < L::kChunks; ++c)
                    tma_load_3d(st + L::kOffV + c * L::kWChunk, &tmV, bar(BAR_WFULL + s), c * 64, row, hk);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc1 = umma_idesc(128, 2 * kBI, false, false);  // S = Q [K;U]^T
            constexpr uint32_t idesc2 = umma_idesc(128, DH, false, true);        // O += A V  (V is MN-major)
            auto gemm2 = [&](int jj) -> bool {  // O += A(jj) V(jj)
                const int s = jj % kStages, bb = jj & 1, nb = jj >> 1;
                if (!mbar_wait(bar(BAR_AFULL + bb), nb & 1, ctl, W + 4)) return false;
                tc_fence_after();
                const uint32_t a0 = sA + bb * L::kABytes, v0 = sW + s * L::kStageBytes + L::kOffV;
#pragma unroll
                for (int k = 0; k < kBI / 16; ++k)
                    umma_ss(tmem + kColO, desc_kmajor(a0 + k * 32), desc_mnmajor(v0 + k * 2048, L::kWChunk), idesc2,
                            (jj > 0 || k > 0) ? 1u : 0u);
                umma_commit(bar(BAR_WEMPTY + s));
                umma_commit(bar(BAR_AEMPTY + bb));
                return true;
            };
            bool ok = mbar_wait(bar(BAR_Q), 0, ctl, W + 2);
            for (int j = 0; ok && j < nblk; ++j) {
                const int s = j % kStages, n = j / kStages, bb = j & 1, nb = j >> 1;
                if (!mbar_wait(bar(BAR_WFULL + s), n & 1, ctl, W + 3)) { ok = false; break; }
                if (!mbar_wait(bar(BAR_SEMPTY + bb), (nb & 1) ^ 1, ctl, W + 5)) { ok = false; break; }
                tc_fence_after();
                const uint32_t st = sW + s * L::kStageBytes;
#pragma unroll
                for (int k = 0; k < DH / 16; ++k) {
                    const int c = k >> 2, kk = k & 3;
                    umma_ss(tmem + kColS0 + bb * kColSStride, desc_kmajor(sQ + c * (kBT * 128) + kk * 32),
                            desc_kmajor(st + c * 2 * L::kWChunk + kk * 32), idesc1, k > 0 ? 1u : 0u);
                }
                umma_commit(bar(BAR_SFULL + bb));
                if (j > 0) ok = gemm2(j - 1);
            }
            if (ok) ok = gemm2(nblk - 1);
            umma_commit(bar(BAR_OFULL));
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------------ activation + epilogue
        const int quarter = warp & 3, half = (warp - 4) >> 2;
        const int row = quarter * 32 + lane;
        const int t = t0 + row;
        const bool in_range = t < args.S;
        const float *rrow = args.R + (long long)b * args.r_sb + (long long)h * args.r_sh + (long long)t * args.r_ss;
        const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
        float r_cur = 0.f, r_next = in_range ? __ldg(rrow) : 0.f;  // routing weight, fetched one sub-network ahead
        bool ok = true;
        for (int j = 0; j < nblk; ++j) {
            const int bb = j & 1, nb = j >> 1;
            if (j % blocks_per_e == 0) {
                const int e1 = j / blocks_per_e + 1;
                r_cur = r_next;
                r_next = (in_range && e1 < args.E) ? __ldg(rrow + e1) : 0.f;
            }
            if (!mbar_wait(bar(BAR_SFULL + bb), nb & 1, ctl, W + 6)) { ok = false; break; }
            tc_fence_after();
            uint32_t m[32], n[32];
            const uint32_t ts = lane_base + kColS0 + bb * kColSStride + half * 32;
            tmem_ld32(ts, m);
            tmem_ld32(ts + kBI, n);
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive(bar(BAR_SEMPTY + bb));
            uint32_t a[16];
            const f32x2 half_r = f2_pack(0.5f * r_cur, 0.5f * r_cur);
#pragma unroll
            for (int i = 0; i < 16; ++i)
                a[i] = fwd_act_pair(f2_pack_bits(m[2 * i], m[2 * i + 1]), f2_pack_bits(n[2 * i], n[2 * i + 1]), half_r);
            if (!mbar_wait(bar(BAR_AEMPTY + bb), (nb & 1) ^ 1, ctl, W + 7)) { ok = false; break; }
            const uint32_t arow = sA + bb * L::kABytes;
#pragma unroll
            for (int i = 0; i < 4; ++i)
                st_shared_v4(arow + sw128_offset(row, half * 4 + i), a[4 * i], a[4 * i + 1], a[4 * i + 2], a[4 * i + 3]);
            fence_async_smem();
            mbar_arrive(bar(BAR_AFULL + bb));
        }
        // epilogue: O (fp32, tensor memory) -> bf16 -> shared (over the Q tile) -> TMA store
        if (ok) ok = mbar_wait(bar(BAR_OFULL), 0, ctl, W + 8);
        if (ok) {
            tc_fence_after();
            constexpr int kColsPerHalf = DH / 2;  // 64, 48 or 32 columns per thread
            const int c0 = half * kColsPerHalf;
#pragma unroll
            for (int g = 0; g < kColsPerHalf / 16; ++g) {
                uint32_t o[16];
                tmem_ld16(lane_base + kColO + c0 + g * 16, o);
                tmem_ld_wait();
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
        named_bar_sync(1, kActThreads);
        if (ok && warp == 4 && lane == 0 && !*abort_flag) {
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
    {  // per device, so set on every call (cheap)
        cudaError_t e = cudaFuncSetAttribute(fwd_kernel<DH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::kTotal);
        if (e != cudaSuccess) { set_cuda_error(e, "cudaFuncSetAttribute(fwd_kernel)"); return FLASHMHF_ERR_CUDA; }
    }
    FwdArgs a{static_cast<const float *>(p.R.ptr), p.R.stride[0], p.R.stride[1], p.R.stride[2],
              p.d.S, p.d.E, p.d.De, p.d.H / p.d.Hkuv, device_status_ptr()};
    dim3 grid((p.d.S + kBT - 1) / kBT, p.d.H, p.d.B);
    prof_mark(st, kMarkStart);
    fwd_kernel<DH><<<grid, kThreads, L::kTotal, st>>>(tmQ, tmK, tmU, tmV, tmO, a);
    prof_mark(st, kMarkFwd);
    *n_launch += 1;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_cuda_error(e, "fwd_kernel launch"); return FLASHMHF_ERR_CUDA; }
    return FLASHMHF_OK;
}

}  // namespace

int tc_forward(const flashmhf_fwd_params &p, cudaStream_t st, int *n_launch) {
    switch (p.d.Dh) {
        case 64: return launch_fwd<64>(p, st, n_launch);
        case 96: return launch_fwd<96>(p, st, n_launch);
        case 128: return launch_fwd<128>(p, st, n_launch);
        default: return FLASHMHF_ERR_BAD_SHAPE;
    }
}

}  // namespace fmhf
