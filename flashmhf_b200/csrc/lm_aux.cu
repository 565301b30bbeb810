// Two memory-bound helpers for the decoder LM the FFN layer is measured in (flashmhf_b200/lm.py): rotary
// position embedding and RMSNorm over the hidden size, forward and backward.  They replace chains of
// element-wise library kernels (10 and 8 passes over the activations) by one pass each way.  They follow
// the reference's arithmetic (models/flashmhf/modeling_mhffnmoe.py:82-87 RMSNorm, :178-206 rotary) in
// fp32 with one rounding to bf16 at the end.
#include "kernels.h"
#include "tc_common.cuh"

namespace fmhf {
namespace {

constexpr int kWarpsAux = 8;

__device__ __forceinline__ float warp_sum32(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ void unpack8(const uint4 v, float (&f)[8]) {
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
    f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
    f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    return make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
}

// ---- rotary: y1 = x1 c - sign x2 s ; y2 = x2 c + sign x1 s  (sign = -1 gives the transpose = backward) ----
// One thread rotates 8 pairs (x1[i..i+7], x2[i..i+7]) of one head of one token.
__global__ void __launch_bounds__(256)
rope_kernel(const __nv_bfloat16 *X, __nv_bfloat16 *Y, const float *cosT, const float *sinT, long long n_items, int S,
            int heads, int hd, long long x_tok, long long y_tok, float sign) {
    const int per_head = hd / 16;   // threads per (token, head)
    for (long long it = (long long)blockIdx.x * blockDim.x + threadIdx.x; it < n_items; it += (long long)gridDim.x * blockDim.x) {
        const int i8 = (int)(it % per_head);
        const long long th = it / per_head;
        const int head = (int)(th % heads);
        const long long t = th / heads;
        const int s = (int)(t % S);
        const __nv_bfloat16 *x = X + t * x_tok + (long long)head * hd + i8 * 8;
        __nv_bfloat16 *y = Y + t * y_tok + (long long)head * hd + i8 * 8;
        float a[8], b[8], c[8], sn[8], o1[8], o2[8];
        unpack8(__ldg(reinterpret_cast<const uint4 *>(x)), a);
        unpack8(__ldg(reinterpret_cast<const uint4 *>(x + hd / 2)), b);
        const float4 *cp = reinterpret_cast<const float4 *>(cosT + (long long)s * (hd / 2) + i8 * 8);
        const float4 *sp = reinterpret_cast<const float4 *>(sinT + (long long)s * (hd / 2) + i8 * 8);
        const float4 c0 = __ldg(cp), c1 = __ldg(cp + 1), s0 = __ldg(sp), s1 = __ldg(sp + 1);
        c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w; c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
        sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float ss = sign * sn[k];
            o1[k] = a[k] * c[k] - b[k] * ss;
            o2[k] = b[k] * c[k] + a[k] * ss;
        }
        *reinterpret_cast<uint4 *>(y) = pack8(o1);
        *reinterpret_cast<uint4 *>(y + hd / 2) = pack8(o2);
    }
}

// ---- RMSNorm over rows of N = 256*CPL elements: one warp per row, lane l holds 16-byte chunks i*32 + l ----
template <int CPL>
__global__ void __launch_bounds__(kWarpsAux * 32)
rmsnorm_fwd_kernel(const __nv_bfloat16 *X, const float *W, __nv_bfloat16 *Y, long long rows, float eps) {
    constexpr int N = CPL * 256;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float w[CPL][8];
#pragma unroll
    for (int i = 0; i < CPL; ++i)
#pragma unroll
        for (int k = 0; k < 8; ++k) w[i][k] = W[(i * 32 + lane) * 8 + k];
    for (long long r = (long long)blockIdx.x * kWarpsAux + warp; r < rows; r += (long long)gridDim.x * kWarpsAux) {
        const uint4 *xr = reinterpret_cast<const uint4 *>(X + r * N);
        float x[CPL][8], ss = 0.f;
#pragma unroll
        for (int i = 0; i < CPL; ++i) {
            unpack8(__ldg(xr + i * 32 + lane), x[i]);
#pragma unroll
            for (int k = 0; k < 8; ++k) ss = fmaf(x[i][k], x[i][k], ss);
        }
        const float rstd = rsqrtf(warp_sum32(ss) * (1.f / (float)N) + eps);
        uint4 *yr = reinterpret_cast<uint4 *>(Y + r * N);
#pragma unroll
        for (int i = 0; i < CPL; ++i) {
            float o[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) o[k] = x[i][k] * rstd * w[i][k];
            yr[i * 32 + lane] = pack8(o);
        }
    }
}

// dx = rstd w g - rstd^3 x mean(w g x) ;  dw += g x rstd  (per-block partial sums, reduced in a second kernel)
template <int CPL>
__global__ void __launch_bounds__(kWarpsAux * 32)
rmsnorm_bwd_kernel(const __nv_bfloat16 *X, const float *W, const __nv_bfloat16 *G, __nv_bfloat16 *dX, float *part_w,
                   long long rows, float eps) {
    constexpr int N = CPL * 256;
    extern __shared__ float sm_aux[];   // [kWarpsAux][N]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float w[CPL][8], wacc[CPL][8];
#pragma unroll
    for (int i = 0; i < CPL; ++i)
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            w[i][k] = W[(i * 32 + lane) * 8 + k];
            wacc[i][k] = 0.f;
        }
    for (long long r = (long long)blockIdx.x * kWarpsAux + warp; r < rows; r += (long long)gridDim.x * kWarpsAux) {
        const uint4 *xr = reinterpret_cast<const uint4 *>(X + r * N), *gr = reinterpret_cast<const uint4 *>(G + r * N);
        float x[CPL][8], g[CPL][8], ss = 0.f, c = 0.f;
#pragma unroll
        for (int i = 0; i < CPL; ++i) {
            unpack8(__ldg(xr + i * 32 + lane), x[i]);
            unpack8(__ldg(gr + i * 32 + lane), g[i]);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                ss = fmaf(x[i][k], x[i][k], ss);
                c = fmaf(w[i][k] * g[i][k], x[i][k], c);
            }
        }
        const float rstd = rsqrtf(warp_sum32(ss) * (1.f / (float)N) + eps);
        const float r3c = rstd * rstd * rstd * warp_sum32(c) * (1.f / (float)N);
        uint4 *dr = reinterpret_cast<uint4 *>(dX + r * N);
#pragma unroll
        for (int i = 0; i < CPL; ++i) {
            float o[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                o[k] = rstd * w[i][k] * g[i][k] - r3c * x[i][k];
                wacc[i][k] = fmaf(g[i][k] * x[i][k], rstd, wacc[i][k]);
            }
            dr[i * 32 + lane] = pack8(o);
        }
    }
#pragma unroll
    for (int i = 0; i < CPL; ++i)
#pragma unroll
        for (int k = 0; k < 8; ++k) sm_aux[warp * N + (i * 32 + lane) * 8 + k] = wacc[i][k];
    __syncthreads();
    for (int j = threadIdx.x; j < N; j += blockDim.x) {
        float v = 0.f;
#pragma unroll
        for (int wp = 0; wp < kWarpsAux; ++wp) v += sm_aux[wp * N + j];
        part_w[(long long)blockIdx.x * N + j] = v;
    }
}

__global__ void __launch_bounds__(128) aux_reduce_kernel(const float *part, float *out, int n, int nblk) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = 0.f;
    for (int b = 0; b < nblk; ++b) v += part[(long long)b * n + i];
    out[i] = v;
}

int norm_blocks(long long rows) {
    const long long most = (rows + kWarpsAux - 1) / kWarpsAux, want = 2 * num_sms();
    return (int)(want < most ? want : most);
}
bool norm_ok(long long rows, int n) { return rows >= 1 && (n == 768 || n == 1024 || n == 2048); }
bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

int lm_rope(const void *x, void *y, const float *cos_t, const float *sin_t, long long tokens, int S, int heads, int hd,
            long long x_tok, long long y_tok, int transpose, cudaStream_t st, int *n_launch) {
    if (!x || !y || !cos_t || !sin_t) return FLASHMHF_ERR_NULL;
    if (tokens < 1 || S < 1 || heads < 1 || hd < 16 || (hd % 16) != 0) return FLASHMHF_ERR_BAD_SHAPE;
    if ((x_tok & 7) || (y_tok & 7) || x_tok < (long long)heads * hd || y_tok < (long long)heads * hd || !aligned16(x) ||
        !aligned16(y) || !aligned16(cos_t) || !aligned16(sin_t))
        return FLASHMHF_ERR_BAD_STRIDE;
    const long long items = tokens * heads * (hd / 16);
    const long long blocks = (items + 255) / 256;
    const long long cap = 8LL * num_sms();
    const int grid = (int)(blocks < cap ? blocks : cap);
    rope_kernel<<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(x), static_cast<__nv_bfloat16 *>(y), cos_t, sin_t,
                                     items, S, heads, hd, x_tok, y_tok, transpose ? -1.f : 1.f);
    *n_launch += 1;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_cuda_error(e, "rope_kernel launch"); return FLASHMHF_ERR_CUDA; }
    return FLASHMHF_OK;
}

int lm_rmsnorm_forward(const void *x, const float *w, void *y, long long rows, int n, float eps, cudaStream_t st, int *n_launch) {
    if (!x || !w || !y) return FLASHMHF_ERR_NULL;
    if (!norm_ok(rows, n)) return FLASHMHF_ERR_BAD_SHAPE;
    if (!aligned16(x) || !aligned16(y)) return FLASHMHF_ERR_BAD_STRIDE;
    const int grid = norm_blocks(rows);
    const __nv_bfloat16 *X = static_cast<const __nv_bfloat16 *>(x);
    __nv_bfloat16 *Y = static_cast<__nv_bfloat16 *>(y);
    if (n == 768) rmsnorm_fwd_kernel<3><<<grid, kWarpsAux * 32, 0, st>>>(X, w, Y, rows, eps);
    else if (n == 1024) rmsnorm_fwd_kernel<4><<<grid, kWarpsAux * 32, 0, st>>>(X, w, Y, rows, eps);
    else rmsnorm_fwd_kernel<8><<<grid, kWarpsAux * 32, 0, st>>>(X, w, Y, rows, eps);
    *n_launch += 1;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_cuda_error(e, "rmsnorm_fwd_kernel launch"); return FLASHMHF_ERR_CUDA; }
    return FLASHMHF_OK;
}

size_t lm_rmsnorm_backward_workspace_bytes(long long rows, int n) {
    return norm_ok(rows, n) ? (size_t)norm_blocks(rows) * (size_t)n * sizeof(float) : 0;
}

int lm_rmsnorm_backward(const void *x, const float *w, const void *g, void *dx, float *dw, void *workspace,
                        size_t workspace_bytes, long long rows, int n, float eps, cudaStream_t st, int *n_launch) {
    if (!x || !w || !g || !dx || !dw) return FLASHMHF_ERR_NULL;
    if (!norm_ok(rows, n)) return FLASHMHF_ERR_BAD_SHAPE;
    if (!aligned16(x) || !aligned16(g) || !aligned16(dx)) return FLASHMHF_ERR_BAD_STRIDE;
    if (!workspace || workspace_bytes < lm_rmsnorm_backward_workspace_bytes(rows, n) || !aligned16(workspace))
        return FLASHMHF_ERR_WORKSPACE;
    const int grid = norm_blocks(rows);
    const size_t smem = (size_t)kWarpsAux * n * sizeof(float);
    const __nv_bfloat16 *X = static_cast<const __nv_bfloat16 *>(x), *G = static_cast<const __nv_bfloat16 *>(g);
    __nv_bfloat16 *dX = static_cast<__nv_bfloat16 *>(dx);
    float *part = static_cast<float *>(workspace);
    cudaError_t e = cudaSuccess;
    if (n == 768) {
        rmsnorm_bwd_kernel<3><<<grid, kWarpsAux * 32, smem, st>>>(X, w, G, dX, part, rows, eps);
    } else if (n == 1024) {
        rmsnorm_bwd_kernel<4><<<grid, kWarpsAux * 32, smem, st>>>(X, w, G, dX, part, rows, eps);
    } else {
        e = cudaFuncSetAttribute(rmsnorm_bwd_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) rmsnorm_bwd_kernel<8><<<grid, kWarpsAux * 32, smem, st>>>(X, w, G, dX, part, rows, eps);
    }
    *n_launch += 1;
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) { set_cuda_error(e, "rmsnorm_bwd_kernel launch"); return FLASHMHF_ERR_CUDA; }
    aux_reduce_kernel<<<(n + 127) / 128, 128, 0, st>>>(part, dw, n, grid);
    *n_launch += 1;
    if ((e = cudaGetLastError()) != cudaSuccess) { set_cuda_error(e, "aux_reduce_kernel launch"); return FLASHMHF_ERR_CUDA; }
    return FLASHMHF_OK;
}

}  // namespace fmhf
