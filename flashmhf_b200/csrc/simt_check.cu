// fp32 check kernels: the operator and its gradients on CUDA cores, fp32 throughout, one warp per
// token row (forward, dQ/dR) or per weight row (dK/dU/dV).  They exist to pin the math of the
// tensor-core kernels on the device (same entry points, dtype = FLASHMHF_F32_CHECK) at the
// tolerance an fp32 evaluation allows; they are not a performance path.
//
// Math (per sub-network e, r = R[..., e]):
//   M = Q K_e^T, N = Q U_e^T, sg = sigmoid(M), s = M*sg, A = s*N*r, O += A V_e
//   dA = dO V_e^T, dR_e = sum_j dA*s*N, dM = dA*(r*N)*(sg + s*(1-sg)), dN = dA*s*r
//   dQ += dM K_e + dN U_e ; dK_e = sum_t dM^T Q ; dU_e = sum_t dN^T Q ; dV_e = sum_t A^T dO
#include "kernels.h"

namespace fmhf {
namespace {

constexpr int kMaxNQ = 4;  // d_h <= 128 -> at most 4 values per lane

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

struct Dims {
    int B, H, S, Dh, Hkuv, E, De, G;
    float s0, s1, s2;  // head, up and final scaling:  M = s0 Q K^T,  N = s1 Q U^T,  A = silu(M) N r s2
};

struct T4 {
    const float *p;
    long long s0, s1, s2;
};

__global__ void __launch_bounds__(256) simt_fwd_kernel(Dims d, T4 Q, T4 K, T4 U, T4 V, T4 R, float *O, long long o0,
                                                       long long o1, long long o2) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const long long rows = (long long)d.B * d.H * d.S;
    if (warp >= rows) return;
    const int t = warp % d.S, h = (warp / d.S) % d.H, b = warp / (d.S * d.H), hk = h / d.G;
    const float *q = Q.p + b * Q.s0 + h * Q.s1 + t * Q.s2;
    const float *r = R.p + b * R.s0 + h * R.s1 + t * R.s2;
    float qv[kMaxNQ], acc[kMaxNQ];
#pragma unroll
    for (int i = 0; i < kMaxNQ; ++i) {
        int c = lane + 32 * i;
        qv[i] = c < d.Dh ? q[c] : 0.f;
        acc[i] = 0.f;
    }
    for (int e = 0; e < d.E; ++e) {
        const float re = r[e];
        for (int j = 0; j < d.De; ++j) {
            const float *k = K.p + hk * K.s0 + e * K.s1 + j * K.s2;
            const float *u = U.p + hk * U.s0 + e * U.s1 + j * U.s2;
            const float *v = V.p + hk * V.s0 + e * V.s1 + j * V.s2;
            float m = 0.f, n = 0.f, vv[kMaxNQ];
#pragma unroll
            for (int i = 0; i < kMaxNQ; ++i) {
                int c = lane + 32 * i;
                bool ok = c < d.Dh;
                m += qv[i] * (ok ? k[c] : 0.f);
                n += qv[i] * (ok ? u[c] : 0.f);
                vv[i] = ok ? v[c] : 0.f;
            }
            m = warp_sum(m) * d.s0;
            n = warp_sum(n) * d.s1;
            const float sg = 1.f / (1.f + expf(-m));
            const float a = m * sg * n * re * d.s2;
#pragma unroll
            for (int i = 0; i < kMaxNQ; ++i) acc[i] += a * vv[i];
        }
    }
    float *o = O + b * o0 + h * o1 + t * o2;
#pragma unroll
    for (int i = 0; i < kMaxNQ; ++i) {
        int c = lane + 32 * i;
        if (c < d.Dh) o[c] = acc[i];
    }
}

__global__ void __launch_bounds__(256) simt_bwd_dq_kernel(Dims d, T4 Q, T4 K, T4 U, T4 V, T4 R, T4 dO, float *dQ,
                                                          long long q0, long long q1, long long q2, float *dR,
                                                          long long r0, long long r1, long long r2) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const long long rows = (long long)d.B * d.H * d.S;
    if (warp >= rows) return;
    const int t = warp % d.S, h = (warp / d.S) % d.H, b = warp / (d.S * d.H), hk = h / d.G;
    const float *q = Q.p + b * Q.s0 + h * Q.s1 + t * Q.s2;
    const float *g = dO.p + b * dO.s0 + h * dO.s1 + t * dO.s2;
    const float *r = R.p + b * R.s0 + h * R.s1 + t * R.s2;
    float qv[kMaxNQ], gv[kMaxNQ], acc[kMaxNQ];
#pragma unroll
    for (int i = 0; i < kMaxNQ; ++i) {
        int c = lane + 32 * i;
        qv[i] = c < d.Dh ? q[c] : 0.f;
        gv[i] = c < d.Dh ? g[c] : 0.f;
        acc[i] = 0.f;
    }
    for (int e = 0; e < d.E; ++e) {
        const float re = r[e];
        float dre = 0.f;
        for (int j = 0; j < d.De; ++j) {
            const float *k = K.p + hk * K.s0 + e * K.s1 + j * K.s2;
            const float *u = U.p + hk * U.s0 + e * U.s1 + j * U.s2;
            const float *v = V.p + hk * V.s0 + e * V.s1 + j * V.s2;
            float m = 0.f, n = 0.f, da = 0.f, kv[kMaxNQ], uv[kMaxNQ];
#pragma unroll
            for (int i = 0; i < kMaxNQ; ++i) {
                int c = lane + 32 * i;
                bool ok = c < d.Dh;
                kv[i] = ok ? k[c] : 0.f;
                uv[i] = ok ? u[c] : 0.f;
                m += qv[i] * kv[i];
                n += qv[i] * uv[i];
                da += gv[i] * (ok ? v[c] : 0.f);
            }
            m = warp_sum(m) * d.s0;
            n = warp_sum(n) * d.s1;
            da = warp_sum(da) * d.s2;   // gradient w.r.t. the unscaled product silu(M) N r
            const float sg = 1.f / (1.f + expf(-m));
            const float s = m * sg;
            dre += da * s * n;
            const float dm = da * (re * n) * (sg + s * (1.f - sg)) * d.s0;  // w.r.t. Q K^T
            const float dn = da * s * re * d.s1;                            // w.r.t. Q U^T
#pragma unroll
            for (int i = 0; i < kMaxNQ; ++i) acc[i] += dm * kv[i] + dn * uv[i];
        }
        if (lane == 0) dR[b * r0 + h * r1 + t * r2 + e] = dre;
    }
    float *o = dQ + b * q0 + h * q1 + t * q2;
#pragma unroll
    for (int i = 0; i < kMaxNQ; ++i) {
        int c = lane + 32 * i;
        if (c < d.Dh) o[c] = acc[i];
    }
}

// One warp per weight row (hk, e, j); walks every token of every query head that shares hk.
__global__ void __launch_bounds__(256) simt_bwd_dw_kernel(Dims d, T4 Q, T4 K, T4 U, T4 V, T4 R, T4 dO, T4 dK, T4 dU,
                                                          T4 dV) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const long long rows = (long long)d.Hkuv * d.E * d.De;
    if (warp >= rows) return;
    const int j = warp % d.De, e = (warp / d.De) % d.E, hk = warp / (d.De * d.E);
    const float *k = K.p + hk * K.s0 + e * K.s1 + j * K.s2;
    const float *u = U.p + hk * U.s0 + e * U.s1 + j * U.s2;
    const float *v = V.p + hk * V.s0 + e * V.s1 + j * V.s2;
    float kv[kMaxNQ], uv[kMaxNQ], vv[kMaxNQ], ak[kMaxNQ], au[kMaxNQ], av[kMaxNQ];
#pragma unroll
    for (int i = 0; i < kMaxNQ; ++i) {
        int c = lane + 32 * i;
        bool ok = c < d.Dh;
        kv[i] = ok ? k[c] : 0.f;
        uv[i] = ok ? u[c] : 0.f;
        vv[i] = ok ? v[c] : 0.f;
        ak[i] = au[i] = av[i] = 0.f;
    }
    for (int b = 0; b < d.B; ++b)
        for (int gi = 0; gi < d.G; ++gi) {
            const int h = hk * d.G + gi;
            for (int t = 0; t < d.S; ++t) {
                const float *q = Q.p + b * Q.s0 + h * Q.s1 + t * Q.s2;
                const float *g = dO.p + b * dO.s0 + h * dO.s1 + t * dO.s2;
                const float re = R.p[b * R.s0 + h * R.s1 + t * R.s2 + e];
                float m = 0.f, n = 0.f, da = 0.f, qv[kMaxNQ], gv[kMaxNQ];
#pragma unroll
                for (int i = 0; i < kMaxNQ; ++i) {
                    int c = lane + 32 * i;
                    bool ok = c < d.Dh;
                    qv[i] = ok ? q[c] : 0.f;
                    gv[i] = ok ? g[c] : 0.f;
                    m += qv[i] * kv[i];
                    n += qv[i] * uv[i];
                    da += gv[i] * vv[i];
                }
                m = warp_sum(m) * d.s0;
                n = warp_sum(n) * d.s1;
                da = warp_sum(da) * d.s2;
                const float sg = 1.f / (1.f + expf(-m));
                const float s = m * sg;
                const float a = s * n * re * d.s2;
                const float dm = da * (re * n) * (sg + s * (1.f - sg)) * d.s0;
                const float dn = da * s * re * d.s1;
#pragma unroll
                for (int i = 0; i < kMaxNQ; ++i) {
                    ak[i] += dm * qv[i];
                    au[i] += dn * qv[i];
                    av[i] += a * gv[i];
                }
            }
        }
    float *ok_ = const_cast<float *>(dK.p) + hk * dK.s0 + e * dK.s1 + j * dK.s2;
    float *ou_ = const_cast<float *>(dU.p) + hk * dU.s0 + e * dU.s1 + j * dU.s2;
    float *ov_ = const_cast<float *>(dV.p) + hk * dV.s0 + e * dV.s1 + j * dV.s2;
#pragma unroll
    for (int i = 0; i < kMaxNQ; ++i) {
        int c = lane + 32 * i;
        if (c < d.Dh) {
            ok_[c] = ak[i];
            ou_[c] = au[i];
            ov_[c] = av[i];
        }
    }
}

T4 t4(const flashmhf_tensor &t) { return T4{static_cast<const float *>(t.ptr), t.stride[0], t.stride[1], t.stride[2]}; }
Dims dims(const flashmhf_dims &d, const flashmhf_scaling &s) {
    return Dims{d.B, d.H, d.S, d.Dh, d.Hkuv, d.E, d.De, d.H / d.Hkuv, s.head_scaling, s.up_scaling, s.final_scaling};
}

}  // namespace

cudaError_t simt_forward(const flashmhf_fwd_params &p, cudaStream_t st, int *n_launch) {
    const long long rows = (long long)p.d.B * p.d.H * p.d.S;
    const unsigned blocks = (unsigned)((rows + 7) / 8);
    simt_fwd_kernel<<<blocks, 256, 0, st>>>(dims(p.d, p.scale), t4(p.Q), t4(p.K), t4(p.U), t4(p.V), t4(p.R),
                                            static_cast<float *>(p.O.ptr), p.O.stride[0], p.O.stride[1], p.O.stride[2]);
    *n_launch += 1;
    return cudaGetLastError();
}

cudaError_t simt_backward(const flashmhf_bwd_params &p, cudaStream_t st, int *n_launch) {
    const long long rows = (long long)p.d.B * p.d.H * p.d.S;
    cudaError_t e = cudaSuccess;
    if (p.parts & FLASHMHF_BWD_INPUTS) {
        simt_bwd_dq_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(
            dims(p.d, p.scale), t4(p.Q), t4(p.K), t4(p.U), t4(p.V), t4(p.R), t4(p.dO), static_cast<float *>(p.dQ.ptr),
            p.dQ.stride[0], p.dQ.stride[1], p.dQ.stride[2], static_cast<float *>(p.dR.ptr), p.dR.stride[0],
            p.dR.stride[1], p.dR.stride[2]);
        *n_launch += 1;
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
    }
    if (p.parts & FLASHMHF_BWD_WEIGHTS) {
        const long long wrows = (long long)p.d.Hkuv * p.d.E * p.d.De;
        simt_bwd_dw_kernel<<<(unsigned)((wrows + 7) / 8), 256, 0, st>>>(dims(p.d, p.scale), t4(p.Q), t4(p.K), t4(p.U),
                                                                       t4(p.V), t4(p.R), t4(p.dO), t4(p.dK), t4(p.dU),
                                                                       t4(p.dV));
        *n_launch += 1;
        e = cudaGetLastError();
    }
    return e;
}

}  // namespace fmhf
