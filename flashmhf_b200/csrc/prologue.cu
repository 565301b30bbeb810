// Fused prologue of the FFN layer: what the reference does between its first projection and the
// operator (models/flashmhf/modeling_mhffnmoe.py:362-386, per-head RMSNorm :116-135), in one pass
// over the projected activations instead of five or six element-wise kernels and two copies:
//
//   X [B,S,H,d_h] (bf16, the projection's own layout)
//     -> per-head RMSNorm in fp32:  y = x * rsqrt(mean_d(x^2) + eps) * w[h,:]      (optional)
//     -> Q = bf16(y), written in the SAME [B,S,H,d_h] layout (the operator reads it through a strided
//        TMA map, so the reference's transpose(1,2).contiguous() copy disappears)
//     -> logits_e = sum_d float(Q_d) * router[h,d,e];  sg = sigmoid(logits)
//     -> R[b,h,s,e] = sg_e / max(sum_e sg_e, 1e-20)                                  (fp32)
//
// and its backward (dQ and dR from the operator -> dX, d router, d w), recomputing the forward from X.
//
// Both are HBM-bound streaming kernels.  Two families share this file's host code:
//   * up to 24 sub-networks per head (the shipped configurations have 8, 11 and 22): prologue_mma.cuh -- 16-token tiles per
//     warp, the three small products as warp-level MMA tiles;
//   * 25..32 sub-networks: the kernels below -- one warp owns one (token, head) row at a time, lane l
//     holds the d_h/32 consecutive elements d = l*d_h/32 .. (one 8-byte load per lane for d_h = 128), the
//     head's router matrix sits re-ordered in shared memory, the logits are reduced across lanes with a
//     transposing butterfly, and the backward keeps its share of d router in registers.
// In both, a block serves one head on a persistent grid (heads x about one or two blocks per SM), loads
// its head's router matrix once and deals tokens to its warps round-robin.  Weight gradients leave the
// block as per-block partial sums and are added over blocks by a second kernel in a fixed order (no
// floating-point atomics, so results are bit-reproducible).
#include "kernels.h"
#include "tc_common.cuh"

namespace fmhf {
namespace {

constexpr int kWarps = 8;             // warps per block
constexpr int kNR = 2;                // rows a warp has in flight
constexpr int kMaxE = 32;
constexpr int kFwdBlocksPerSM = 2;

// Row pair q of warp `warp` in block column `by` of `gy`: pairs are dealt round-robin over warps, then blocks.
__device__ __forceinline__ long long first_row(int q, int by, int gy, int warp) {
    return (long long)kNR * (((long long)q * gy + by) * kWarps + warp);
}

struct ProArgs {
    const __nv_bfloat16 *X;   // [B,S,H,Dh]
    long long x_tok;          // element stride between tokens (= H*Dh when contiguous)
    const float *W;           // [H,Dh] or nullptr (no RMSNorm)
    const float *router;      // [H,Dh,E]
    float eps;
    int T, H, E, S;           // T = B*S tokens
    unsigned s_mul, s_shift;  // t / S == (t * s_mul) >> s_shift for 0 <= t < 2^31
};

// Division of a token index by the sequence length without the 64-bit divide: round-up multiplier.
__device__ __forceinline__ int div_by_s(long long t, const ProArgs &a) {
    return (int)(((unsigned long long)(unsigned)t * a.s_mul) >> a.s_shift);
}

template <int N>
__device__ __forceinline__ float group_sum(float v) {  // sum over aligned groups of N lanes
#pragma unroll
    for (int o = N / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// p[e], e < EP, are per-lane partial sums.  Returns, in every lane l, the sum over all 32 lanes of
// p[l % EP]: EP-1 exchange steps that halve the live values, then plain butterflies across the groups.
template <int EP>
__device__ __forceinline__ float reduce_transpose(float (&p)[EP], int lane) {
#pragma unroll
    for (int off = EP / 2; off >= 1; off >>= 1) {
        const bool up = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < off; ++i) {
            const float lo = p[i], hi = p[i + off];
            const float recv = __shfl_xor_sync(0xffffffffu, up ? lo : hi, off);
            p[i] = (up ? hi : lo) + recv;
        }
    }
    float v = p[0];
#pragma unroll
    for (int off = EP; off < 32; off <<= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// EPL consecutive bf16 of one row <-> floats.  The row pointer is 8-byte aligned for EPL = 4 and
// 4-byte aligned for EPL = 2 (checked on the host).
template <int EPL>
__device__ __forceinline__ void load_row(const __nv_bfloat16 *row, int lane, bool ok, float (&x)[EPL]) {
    if (!ok) {
#pragma unroll
        for (int i = 0; i < EPL; ++i) x[i] = 0.f;
        return;
    }
    if constexpr (EPL == 4) {
        const uint2 v = __ldg(reinterpret_cast<const uint2 *>(row) + lane);
        x[0] = __uint_as_float(v.x << 16); x[1] = __uint_as_float(v.x & 0xffff0000u);
        x[2] = __uint_as_float(v.y << 16); x[3] = __uint_as_float(v.y & 0xffff0000u);
    } else if constexpr (EPL == 2) {
        const uint32_t v = __ldg(reinterpret_cast<const uint32_t *>(row) + lane);
        x[0] = __uint_as_float(v << 16); x[1] = __uint_as_float(v & 0xffff0000u);
    } else {
#pragma unroll
        for (int i = 0; i < EPL; ++i) x[i] = __bfloat162float(row[lane * EPL + i]);
    }
}
template <int EPL>
__device__ __forceinline__ void store_row(__nv_bfloat16 *row, int lane, const float (&x)[EPL]) {
    if constexpr (EPL == 4) {
        uint2 v;
        v.x = pack_bf16(x[0], x[1]);
        v.y = pack_bf16(x[2], x[3]);
        reinterpret_cast<uint2 *>(row)[lane] = v;
    } else if constexpr (EPL == 2) {
        reinterpret_cast<uint32_t *>(row)[lane] = pack_bf16(x[0], x[1]);
    } else {
#pragma unroll
        for (int i = 0; i < EPL; ++i) row[lane * EPL + i] = __float2bfloat16(x[i]);
    }
}
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16(v)); }

// The router slice of one lane, router[h, lane*EPL + i, e], in shared memory as [e][i][lane] (conflict-free):
// these kernels serve 25..32 sub-networks, where a register copy next to the backward's same-shaped accumulator
// would not fit (up to 24 sub-networks run the MMA kernels of prologue_mma.cuh).
template <int EPL, int EP>
struct RouterSlice {
    const float *sm;
    int lane;
    // Stages router[h] (Dh*E floats) in shared memory with coalesced loads, then re-orders it.  `stage`: 2*Dh*E floats.
    __device__ __forceinline__ void init(const float *router_h, float *stage, int E, int lane_) {
        lane = lane_;
        const int n = EPL * 32 * E;
        for (int k = threadIdx.x; k < n; k += blockDim.x) stage[k] = router_h[k];
        __syncthreads();
        float *dst = stage + n;
        for (int k = threadIdx.x; k < n; k += blockDim.x) {
            const int d = k / E, e = k - d * E;  // d = l*EPL + i
            dst[(e * EPL + d % EPL) * 32 + d / EPL] = stage[k];
        }
        sm = dst;
        __syncthreads();
    }
    __device__ __forceinline__ float at(int i, int e) const { return sm[(e * EPL + i) * 32 + lane]; }
};

template <int EPL>
struct Row {
    float x[EPL], y[EPL];  // input; what the router and the operator see (bf16-rounded when normalised)
    float rstd, sg, D;     // sg: sigmoid of the logit of sub-network lane % EP (0 beyond E)
};

template <int DH, int EP, bool NORM>
__device__ __forceinline__ void row_forward(Row<DH / 32> &r, const float (&w)[DH / 32], const RouterSlice<DH / 32, EP> &rt,
                                            float eps, int E, int lane) {
    constexpr int EPL = DH / 32;
    if (NORM) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) ss = fmaf(r.x[i], r.x[i], ss);
        ss = group_sum<32>(ss);
        r.rstd = rsqrtf(ss * (1.f / (float)DH) + eps);
#pragma unroll
        for (int i = 0; i < EPL; ++i) r.y[i] = bf16_round(r.x[i] * r.rstd * w[i]);
    } else {
        r.rstd = 1.f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) r.y[i] = r.x[i];
    }
    float part[EP];
#pragma unroll
    for (int e = 0; e < EP; ++e) {
        float v = 0.f;
        if (e < E) {
#pragma unroll
            for (int i = 0; i < EPL; ++i) v = fmaf(r.y[i], rt.at(i, e), v);
        }
        part[e] = v;
    }
    const float logit = reduce_transpose<EP>(part, lane);
    r.sg = (lane & (EP - 1)) < E ? __fdividef(1.f, 1.f + __expf(-logit)) : 0.f;
    r.D = fmaxf(group_sum<EP>(r.sg), 1e-20f);
}

template <int DH, int EP, bool NORM>
__global__ void __launch_bounds__(kWarps * 32, 2)
prologue_fwd_kernel(const ProArgs a, __nv_bfloat16 *Q, float *R) {
    constexpr int EPL = DH / 32;
    extern __shared__ float sm[];
    const int h = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    RouterSlice<EPL, EP> rt;
    rt.init(a.router + (long long)h * DH * a.E, sm, a.E, lane);
    float w[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) w[i] = NORM ? a.W[h * DH + lane * EPL + i] : 1.f;

    const int by = blockIdx.y, gy = gridDim.y;
    float xn[kNR][EPL];
    long long t = first_row(0, by, gy, warp);
#pragma unroll
    for (int k = 0; k < kNR; ++k) load_row<EPL>(a.X + (t + k) * a.x_tok + h * DH, lane, t + k < a.T, xn[k]);
    for (int q = 0; t < a.T; ++q) {
        const long long tn = first_row(q + 1, by, gy, warp);
        Row<EPL> r[kNR];
#pragma unroll
        for (int k = 0; k < kNR; ++k) {
#pragma unroll
            for (int i = 0; i < EPL; ++i) r[k].x[i] = xn[k][i];
            load_row<EPL>(a.X + (tn + k) * a.x_tok + h * DH, lane, tn + k < a.T, xn[k]);
        }
#pragma unroll
        for (int k = 0; k < kNR; ++k) row_forward<DH, EP, NORM>(r[k], w, rt, a.eps, a.E, lane);
#pragma unroll
        for (int k = 0; k < kNR; ++k) {
            const long long tk = t + k;
            if (tk < a.T) {
                if (NORM) store_row<EPL>(Q + tk * a.x_tok + h * DH, lane, r[k].y);
                const long long b = div_by_s(tk, a), s = tk - b * a.S;
                if (lane < a.E) R[((b * a.H + h) * a.S + s) * a.E + lane] = __fdividef(r[k].sg, r[k].D);
            }
        }
        t = tn;
    }
}

struct ProBwdArgs {
    const __nv_bfloat16 *dQ;     // gradient w.r.t. Q as the operator returns it: element strides below
    long long dq_b, dq_h, dq_s;
    const float *dR;             // [B,H,S,E] contiguous
    __nv_bfloat16 *dX;           // [B,S,H,Dh], token stride x_tok
    float *part_router;          // [gridDim.y][H][Dh*E] block partial sums
    float *part_w;               // [gridDim.y][H][Dh]
};

template <int DH, int EP, bool NORM>
__global__ void __launch_bounds__(kWarps * 32, 1)
prologue_bwd_kernel(const ProArgs a, const ProBwdArgs g) {
    constexpr int EPL = DH / 32;
    extern __shared__ float sm[];
    const int E = a.E, DE = DH * E;
    // shared: [router staging and re-ordered copy: 2*DE]
    //         [per-warp d router: kWarps*DE] [per-warp d w: kWarps*DH]
    float *router_s = sm;
    float *acc_r = sm + 2 * DE, *acc_w = acc_r + kWarps * DE;
    const int h = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    RouterSlice<EPL, EP> rt;
    rt.init(a.router + (long long)h * DE, router_s, E, lane);
    float w[EPL], wacc[EPL], racc[EPL][EP];
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        w[i] = NORM ? a.W[h * DH + lane * EPL + i] : 1.f;
        wacc[i] = 0.f;
#pragma unroll
        for (int e = 0; e < EP; ++e) racc[i][e] = 0.f;
    }

    const int by = blockIdx.y, gy = gridDim.y;
    float xn[kNR][EPL], qn[kNR][EPL], gn[kNR];
    auto prefetch = [&](int k, long long tt) {
        const bool ok = tt < a.T;
        const long long b = ok ? div_by_s(tt, a) : 0, s = ok ? tt - b * a.S : 0;
        load_row<EPL>(a.X + tt * a.x_tok + h * DH, lane, ok, xn[k]);
        load_row<EPL>(g.dQ + b * g.dq_b + (long long)h * g.dq_h + s * g.dq_s, lane, ok, qn[k]);
        gn[k] = ok && lane < E ? __ldg(g.dR + ((b * a.H + h) * a.S + s) * E + lane) : 0.f;
    };
    long long t = first_row(0, by, gy, warp);
#pragma unroll
    for (int k = 0; k < kNR; ++k) prefetch(k, t + k);

    for (int q = 0; t < a.T; ++q) {
        const long long tn = first_row(q + 1, by, gy, warp);
        Row<EPL> r[kNR];
        float dy[kNR][EPL], ge[kNR];
#pragma unroll
        for (int k = 0; k < kNR; ++k) {
#pragma unroll
            for (int i = 0; i < EPL; ++i) { r[k].x[i] = xn[k][i]; dy[k][i] = qn[k][i]; }
            ge[k] = gn[k];
            prefetch(k, tn + k);
        }
#pragma unroll
        for (int k = 0; k < kNR; ++k) row_forward<DH, EP, NORM>(r[k], w, rt, a.eps, E, lane);
#pragma unroll
        for (int k = 0; k < kNR; ++k) {
            // R_e = sg_e / D  ->  d sg_e = (g_e - sum_k g_k R_k) / D ;  d logit_e = d sg_e * sg_e * (1 - sg_e).
            // A clamped denominator (D = 1e-20) has no gradient through the sum, as torch's clamp.
            const float inv = __fdividef(1.f, r[k].D);
            const float gR = r[k].D > 1e-20f ? group_sum<EP>(ge[k] * r[k].sg * inv) : 0.f;
            const float dl = (ge[k] - gR) * inv * r[k].sg * (1.f - r[k].sg);   // 0 for lanes beyond E (sg = 0)
            // dy = dQ + router . dlogits ;  d router += y (x) dlogits
#pragma unroll
            for (int e = 0; e < EP; ++e) {
                if (e < E) {
                    const float dle = __shfl_sync(0xffffffffu, dl, e);
#pragma unroll
                    for (int i = 0; i < EPL; ++i) {
                        dy[k][i] = fmaf(rt.at(i, e), dle, dy[k][i]);
                        racc[i][e] = fmaf(r[k].y[i], dle, racc[i][e]);
                    }
                }
            }
            // RMSNorm: y_d = w_d x_d rstd ;  dx_d = rstd w_d dy_d - rstd^3 x_d mean_k(w_k dy_k x_k) ;  dw_d += dy_d x_d rstd
            float dx[EPL];
            if (NORM) {
                float c = 0.f;
#pragma unroll
                for (int i = 0; i < EPL; ++i) {
                    c = fmaf(w[i] * dy[k][i], r[k].x[i], c);
                    wacc[i] = fmaf(dy[k][i] * r[k].x[i], r[k].rstd, wacc[i]);
                }
                c = group_sum<32>(c) * (1.f / (float)DH);
                const float r3c = r[k].rstd * r[k].rstd * r[k].rstd * c;
#pragma unroll
                for (int i = 0; i < EPL; ++i) dx[i] = r[k].rstd * w[i] * dy[k][i] - r3c * r[k].x[i];
            } else {
#pragma unroll
                for (int i = 0; i < EPL; ++i) dx[i] = dy[k][i];
            }
            if (t + k < a.T) store_row<EPL>(g.dX + (t + k) * a.x_tok + h * DH, lane, dx);
        }
        t = tn;
    }
    // warps' accumulators -> shared -> this block's partial sums (fixed order)
    float *my_r = acc_r + warp * DE, *my_w = acc_w + warp * DH;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        my_w[lane * EPL + i] = wacc[i];
#pragma unroll
        for (int e = 0; e < EP; ++e)
            if (e < E) my_r[(lane * EPL + i) * E + e] = racc[i][e];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < DE; i += blockDim.x) {
        float v = 0.f;
#pragma unroll
        for (int wp = 0; wp < kWarps; ++wp) v += acc_r[wp * DE + i];
        g.part_router[((long long)blockIdx.y * a.H + h) * DE + i] = v;
    }
    if (NORM)
        for (int i = threadIdx.x; i < DH; i += blockDim.x) {
            float v = 0.f;
#pragma unroll
            for (int wp = 0; wp < kWarps; ++wp) v += acc_w[wp * DH + i];
            g.part_w[((long long)blockIdx.y * a.H + h) * DH + i] = v;
        }
}

#include "prologue_mma.cuh"

// out[i] = sum over blocks (in index order) of part[blk][i]
__global__ void __launch_bounds__(128) prologue_reduce_kernel(const float *part, float *out, long long n, int nblk) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = 0.f;
    int b = 0;
    for (; b + 8 <= nblk; b += 8) {
        float u[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) u[k] = part[(long long)(b + k) * n + i];
#pragma unroll
        for (int k = 0; k < 8; ++k) v += u[k];
    }
    for (; b < nblk; ++b) v += part[(long long)b * n + i];
    out[i] = v;
}

int check_pro(const flashmhf_prologue_params &p, bool forward) {
    if (p.B < 1 || p.S < 1 || p.H < 1 || p.E < 1 || p.E > kMaxE) return FLASHMHF_ERR_BAD_SHAPE;
    if (p.Dh != 64 && p.Dh != 96 && p.Dh != 128) return FLASHMHF_ERR_BAD_SHAPE;
    if ((long long)p.B * p.S > 0x7fffffffLL) return FLASHMHF_ERR_BAD_SHAPE;
    if (!p.X || !p.router) return FLASHMHF_ERR_NULL;
    if (forward && (!p.R || (p.norm_weight && !p.Q))) return FLASHMHF_ERR_NULL;   // the backward call writes neither
    if (p.x_token_stride < (int64_t)p.H * p.Dh || (p.x_token_stride & 7)) return FLASHMHF_ERR_BAD_STRIDE;
    if ((reinterpret_cast<uintptr_t>(p.X) & 15u) || (forward && p.norm_weight && (reinterpret_cast<uintptr_t>(p.Q) & 15u)))
        return FLASHMHF_ERR_BAD_STRIDE;
    return FLASHMHF_OK;
}
ProArgs pro_args(const flashmhf_prologue_params &p) {
    // l = ceil(log2 S); m = floor(2^(31+l) / S) + 1 < 2^32 gives exact quotients for dividends below 2^31
    unsigned l = 0;
    while ((1ull << l) < (unsigned long long)p.S) ++l;
    const unsigned mul = (unsigned)(((1ull << (31 + l)) / (unsigned long long)p.S) + 1ull);
    return ProArgs{static_cast<const __nv_bfloat16 *>(p.X), p.x_token_stride, p.norm_weight, p.router, p.eps,
                   p.B * p.S, p.H, p.E, p.S, mul, 31 + l};
}
// E <= 24 runs the MMA kernels (16-token tiles per warp; the backward's d-router accumulator takes 32 registers per
// 8 sub-networks), more sub-networks the per-lane kernels (row pairs).
bool use_mma(const flashmhf_prologue_params &p) { return p.E <= 24; }

// Blocks per head: enough to fill the GPU `per_sm` times over, never more than there are warp work items to deal.
int blocks_per_head(const flashmhf_prologue_params &p, int per_sm) {
    const int unit = use_mma(p) ? 16 : kNR;
    const long long pairs = ((long long)p.B * p.S + unit - 1) / unit, most = (pairs + kWarps - 1) / kWarps;
    const int sms = num_sms();
    const long long want = sms * per_sm / p.H > 1 ? sms * per_sm / p.H : 1;
    return (int)(want < most ? want : most);
}

size_t fwd_smem(int DH, int EP, int E) { return (size_t)2 * DH * E * sizeof(float); }
size_t bwd_smem(int DH, int EP, int E) {
    return fwd_smem(DH, EP, E) + (size_t)kWarps * ((size_t)DH * E + DH) * sizeof(float);
}

template <int DH, int EP, bool NORM>
cudaError_t launch_fwd(const ProArgs &a, dim3 grid, __nv_bfloat16 *Q, float *R, cudaStream_t st) {
    const size_t smem = fwd_smem(DH, EP, a.E);
    cudaError_t e = cudaFuncSetAttribute(prologue_fwd_kernel<DH, EP, NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    prologue_fwd_kernel<DH, EP, NORM><<<grid, kWarps * 32, smem, st>>>(a, Q, R);
    return cudaGetLastError();
}
template <int DH, int EP, bool NORM>
cudaError_t launch_bwd(const ProArgs &a, dim3 grid, const ProBwdArgs &g, cudaStream_t st) {
    const size_t smem = bwd_smem(DH, EP, a.E);
    cudaError_t e = cudaFuncSetAttribute(prologue_bwd_kernel<DH, EP, NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    prologue_bwd_kernel<DH, EP, NORM><<<grid, kWarps * 32, smem, st>>>(a, g);
    return cudaGetLastError();
}

// dispatch on (d_h, n-tiles of 8 sub-networks, RMSNorm on/off); the per-lane kernels below it serve E > 24
#define FMHF_PRO_DISPATCH_MMA_DH(CALL, DH)                                                  \
    do {                                                                                   \
        const bool norm = p.norm_weight != nullptr;                                        \
        if (p.E <= 8) { if (norm) e = CALL(DH, 1, true); else e = CALL(DH, 1, false); }     \
        else if (p.E <= 16) { if (norm) e = CALL(DH, 2, true); else e = CALL(DH, 2, false); } \
        else { if (norm) e = CALL(DH, 3, true); else e = CALL(DH, 3, false); }              \
    } while (0)
#define FMHF_PRO_DISPATCH_MMA(CALL)                                                        \
    do {                                                                                   \
        if (p.Dh == 128) FMHF_PRO_DISPATCH_MMA_DH(CALL, 128);                              \
        else if (p.Dh == 96) FMHF_PRO_DISPATCH_MMA_DH(CALL, 96);                           \
        else FMHF_PRO_DISPATCH_MMA_DH(CALL, 64);                                           \
    } while (0)

#define FMHF_PRO_DISPATCH(CALL)                                                            \
    do {                                                                                   \
        const bool norm = p.norm_weight != nullptr;                                        \
        if (p.Dh == 128) { if (norm) e = CALL(128, 32, true); else e = CALL(128, 32, false); } \
        else if (p.Dh == 96) { if (norm) e = CALL(96, 32, true); else e = CALL(96, 32, false); } \
        else { if (norm) e = CALL(64, 32, true); else e = CALL(64, 32, false); }            \
    } while (0)

}  // namespace

int prologue_forward(const flashmhf_prologue_params &p, cudaStream_t st, int *n_launch) {
    int rc = check_pro(p, true);
    if (rc) return rc;
    const ProArgs a = pro_args(p);
    const dim3 grid(p.H, blocks_per_head(p, kFwdBlocksPerSM));
    __nv_bfloat16 *Q = static_cast<__nv_bfloat16 *>(p.Q);
    cudaError_t e = cudaSuccess;
    prof_mark(st, kMarkStart);
#define FMHF_FWD(DH, EP, NORM) launch_fwd<DH, EP, NORM>(a, grid, Q, p.R, st)
#define FMHF_FWD_MMA(DH, NT, NORM) launch_fwd_mma<DH, NT, NORM>(a, grid, Q, p.R, st)
    if (use_mma(p)) FMHF_PRO_DISPATCH_MMA(FMHF_FWD_MMA);
    else FMHF_PRO_DISPATCH(FMHF_FWD);
#undef FMHF_FWD
#undef FMHF_FWD_MMA
    prof_mark(st, kMarkPrologueFwd);
    *n_launch += 1;
    if (e != cudaSuccess) { set_cuda_error(e, "prologue_fwd_kernel launch"); return FLASHMHF_ERR_CUDA; }
    return FLASHMHF_OK;
}

size_t prologue_backward_workspace_bytes(const flashmhf_prologue_params &p) {
    return (size_t)blocks_per_head(p, 1) * p.H * ((size_t)p.Dh * p.E + p.Dh) * sizeof(float);
}

int prologue_backward(const flashmhf_prologue_bwd_params &q, cudaStream_t st, int *n_launch) {
    const flashmhf_prologue_params &p = q.fwd;
    int rc = check_pro(p, false);
    if (rc) return rc;
    if (!q.dQ || !q.dR || !q.dX || !q.d_router || (p.norm_weight && !q.d_norm_weight)) return FLASHMHF_ERR_NULL;
    if ((reinterpret_cast<uintptr_t>(q.dQ) & 15u) || (reinterpret_cast<uintptr_t>(q.dX) & 15u) || (q.dq_stride[0] & 7) ||
        (q.dq_stride[1] & 7) || (q.dq_stride[2] & 7))
        return FLASHMHF_ERR_BAD_STRIDE;
    const size_t need = prologue_backward_workspace_bytes(p);
    if (!q.workspace || q.workspace_bytes < need || (reinterpret_cast<uintptr_t>(q.workspace) & 255u))
        return FLASHMHF_ERR_WORKSPACE;
    const ProArgs a = pro_args(p);
    const int ny = blocks_per_head(p, 1), DE = p.Dh * p.E;
    float *part_r = static_cast<float *>(q.workspace);
    float *part_w = part_r + (size_t)ny * p.H * DE;
    const ProBwdArgs g{static_cast<const __nv_bfloat16 *>(q.dQ), q.dq_stride[0], q.dq_stride[1], q.dq_stride[2], q.dR,
                       static_cast<__nv_bfloat16 *>(q.dX), part_r, part_w};
    const dim3 grid(p.H, ny);
    cudaError_t e = cudaSuccess;
    prof_mark(st, kMarkStart);
#define FMHF_BWD(DH, EP, NORM) launch_bwd<DH, EP, NORM>(a, grid, g, st)
#define FMHF_BWD_MMA(DH, NT, NORM) launch_bwd_mma<DH, NT, NORM>(a, grid, g, st)
    if (use_mma(p)) FMHF_PRO_DISPATCH_MMA(FMHF_BWD_MMA);
    else FMHF_PRO_DISPATCH(FMHF_BWD);
#undef FMHF_BWD
#undef FMHF_BWD_MMA
    prof_mark(st, kMarkPrologueBwd);
    *n_launch += 1;
    if (e != cudaSuccess) { set_cuda_error(e, "prologue_bwd_kernel launch"); return FLASHMHF_ERR_CUDA; }
    const long long nr = (long long)p.H * DE, nw = (long long)p.H * p.Dh;
    prologue_reduce_kernel<<<(int)((nr + 127) / 128), 128, 0, st>>>(part_r, q.d_router, nr, ny);
    *n_launch += 1;
    if (p.norm_weight) {
        prologue_reduce_kernel<<<(int)((nw + 127) / 128), 128, 0, st>>>(part_w, q.d_norm_weight, nw, ny);
        *n_launch += 1;
    }
    prof_mark(st, kMarkPrologueReduce);
    if ((e = cudaGetLastError()) != cudaSuccess) { set_cuda_error(e, "prologue_reduce_kernel launch"); return FLASHMHF_ERR_CUDA; }
    return FLASHMHF_OK;
}

}  // namespace fmhf
