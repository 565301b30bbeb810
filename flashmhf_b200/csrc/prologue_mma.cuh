// Prologue kernels for up to 24 sub-networks per head: the three small products of the prologue
//   logits[t,e]    = sum_d y[t,d] router[d,e]                     (forward, and recomputed in backward)
//   dy[t,d]       += sum_e dlogits[t,e] router[d,e]
//   d router[d,e] += sum_t y[t,d] dlogits[t,e]
// run as warp-level 16x8x16 bf16 `mma.sync` tiles with fp32 accumulation instead of per-lane FMAs and a
// cross-lane transposing reduction, which cuts the instructions per (token, head) row by about five.
// These kernels move 0.5-0.8 KB per row and need ~1.4 kFLOP per row for the products: they are bound
// by HBM, the products take a few percent of the tensor pipe, and the register-fragment form needs no
// shared-memory or tensor-memory round trip for its 16-row tiles, so the warp-level instruction is
// the fitting one here (the operator's GEMMs, where throughput matters, use tcgen05).
//
// Exactness: y is bf16 already; the fp32 router and the fp32 dlogits are split into bf16 terms
// (hi + mid + lo, 24 bits) so that products are exact and sums are fp32, as in the fp32 reference math.
//
// Work split: a warp owns 16 consecutive tokens of one head at a time; lane (g = lane/4, q = lane%4) holds
// rows g and g+8 and, of each row, the 16-byte chunks i*4+q (i < d_h/32), i.e. one fully used 64-byte
// segment per row and load instruction.  The MMA's k index is only a summation index, so k-step ks simply
// takes the lane's 32-bit registers 2ks and 2ks+1 and the router fragments are permuted to match (col()).
// Included by prologue.cu inside namespace fmhf::{anonymous}.

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Transposes the 8x8 matrix of bf16 that the warp holds one row-fragment register each of (lane (g,q): row g, columns 2q, 2q+1):
// afterwards the lane holds rows 2q, 2q+1 of column g -- a row-major accumulator-style fragment becomes an operand fragment whose
// k index is the former row index.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t v) {
    uint32_t r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
    return r;
}
// Shared-memory loads the compiler must not hoist out of the tile loop: the fragments are loop-invariant, and kept in
// registers they would cost more than a hundred of them.
__device__ __forceinline__ uint2 lds_u2(const void *p) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(smem_u32(p)));
    return v;
}
__device__ __forceinline__ float2 lds_f2(const void *p) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(smem_u32(p)));
    return v;
}
// 16-byte asynchronous global->shared copy; `ok` false writes zeros and reads nothing.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, bool ok) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(ok ? 16 : 0) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint4 lds_u4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float quad_sum(float v) {  // over the 4 lanes that share a row
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    return v;
}
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

// Memory column of the two bf16 in 32-bit register u of lane quarter q.
__host__ __device__ constexpr int mma_col(int q, int u) { return ((u >> 2) * 4 + q) * 8 + 2 * (u & 3); }

// v = hi + mid + lo with each term a bf16 (lo absorbs what is left; 24 significant bits in all)
__device__ __forceinline__ void split3(float v, float &hi, float &mid, float &lo) {
    hi = bf16_round(v);
    mid = bf16_round(v - hi);
    lo = bf16_round(v - hi - mid);
}

template <int DH, int NT>
struct MmaLayout {
    static constexpr int NI = DH / 32, NU = DH / 8, NKS = DH / 16, NKK = (NT + 1) / 2;
    // shared memory (bytes)
    static constexpr int kBf = 3 * NKS * NT * 32 * 8;        // logits B fragments: [split][ks][nt][lane] (b0, b1)
    static constexpr int kB2f = 2 * NKK * NU * 32 * 8;       // router^T B fragments: [split hi/mid][kk][u][lane]
    static constexpr int kW = DH * 4;
    static constexpr int kOffBf = 0, kOffW = kBf, kOffFwdEnd = kOffW + kW;
    static constexpr int kWacc = 2 * NU * 32 * 4;            // per warp: d norm-weight sums of each lane's 2*NU columns, [u][j][lane]
    // per warp: two stages of {X tile, dQ tile}, 16 rows each, rows padded to DH*2 + 64 bytes so that the two rows a
    // quarter-warp reads with one 16-byte load per lane fall into different banks
    static constexpr int kSRow = DH * 2 + 64, kSTile = 16 * kSRow, kStage = 2 * kSTile;
    static constexpr int kOffB2f = kOffFwdEnd, kOffWacc = kOffB2f + kB2f, kOffStage = kOffWacc + kWarps * kWacc,
                         kOffBwdEnd = kOffStage + kWarps * 2 * kStage;
};

// Router fragments of head h.  Bf feeds logits = y . router (k = d), B2f feeds dy += dlogits . router^T (k = e).
template <int DH, int NT, bool BWD>
__device__ __forceinline__ void build_router_fragments(const float *router_h, int E, uint8_t *smem) {
    using L = MmaLayout<DH, NT>;
    uint2 *bf = reinterpret_cast<uint2 *>(smem + L::kOffBf);
    for (int idx = threadIdx.x; idx < L::NKS * NT * 32; idx += blockDim.x) {
        const int ln = idx & 31, nt = (idx >> 5) % NT, ks = (idx >> 5) / NT;
        const int g = ln >> 2, q = ln & 3, e = nt * 8 + g;
        float v[4], s[3][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {   // (u0,b0) (u0,b1) (u1,b0) (u1,b1)
            const int d = mma_col(q, 2 * ks + (j >> 1)) + (j & 1);
            v[j] = e < E ? router_h[d * E + e] : 0.f;
            split3(v[j], s[0][j], s[1][j], s[2][j]);
        }
#pragma unroll
        for (int t = 0; t < 3; ++t)
            bf[((t * L::NKS + ks) * NT + nt) * 32 + ln] = make_uint2(pack_bf16(s[t][0], s[t][1]), pack_bf16(s[t][2], s[t][3]));
    }
    if (BWD) {
        uint2 *b2 = reinterpret_cast<uint2 *>(smem + L::kOffB2f);
        for (int idx = threadIdx.x; idx < L::NKK * L::NU * 32; idx += blockDim.x) {
            const int ln = idx & 31, u = (idx >> 5) % L::NU, kk = (idx >> 5) / L::NU;
            const int g = ln >> 2, q = ln & 3;
            const int d = mma_col(g >> 1, u) + (g & 1);      // the column that accumulator column g of n-tile u stands for
            float hi[4], mid[4], lo;
#pragma unroll
            for (int j = 0; j < 4; ++j) {   // experts kk*16 + 2q + {0,1}, then + 8
                const int e = kk * 16 + (j >> 1) * 8 + 2 * q + (j & 1);
                const float v = e < E ? router_h[d * E + e] : 0.f;
                split3(v, hi[j], mid[j], lo);
            }
            b2[((0 * L::NKK + kk) * L::NU + u) * 32 + ln] = make_uint2(pack_bf16(hi[0], hi[1]), pack_bf16(hi[2], hi[3]));
            b2[((1 * L::NKK + kk) * L::NU + u) * 32 + ln] = make_uint2(pack_bf16(mid[0], mid[1]), pack_bf16(mid[2], mid[3]));
        }
    }
}

// Rows g and g+8 of a 16-token tile: load, per-head RMSNorm, logits by MMA, sigmoid and normalisation.
template <int DH, int NT>
struct MmaRows {
    static constexpr int NU = DH / 8;
    uint32_t x[2][NU];      // bf16 pairs as loaded
    uint32_t y[2][NU];      // what the router and the operator see
    float rstd[2], sg[NT][4], D[2];   // sg[nt][j]: row j>>1, sub-network nt*8 + 2q + (j&1)
};

template <int DH, int NT, bool NORM>
__device__ __forceinline__ void mma_rows_forward(MmaRows<DH, NT> &r, const ProArgs &a, const uint8_t *smem, int lane) {
    using L = MmaLayout<DH, NT>;
    const int q = lane & 3;
    const float *wsm = reinterpret_cast<const float *>(smem + L::kOffW);
    if (NORM) {
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            float ss = 0.f;
#pragma unroll
            for (int u = 0; u < L::NU; ++u) {
                const float lo = bf16_lo(r.x[k][u]), hi = bf16_hi(r.x[k][u]);
                ss = fmaf(lo, lo, fmaf(hi, hi, ss));
            }
            r.rstd[k] = rsqrtf(quad_sum(ss) * (1.f / (float)DH) + a.eps);
        }
#pragma unroll
        for (int u = 0; u < L::NU; ++u) {
            const float2 w = lds_f2(wsm + mma_col(q, u));
#pragma unroll
            for (int k = 0; k < 2; ++k)
                r.y[k][u] = pack_bf16(bf16_lo(r.x[k][u]) * r.rstd[k] * w.x, bf16_hi(r.x[k][u]) * r.rstd[k] * w.y);
        }
    } else {
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            r.rstd[k] = 1.f;
#pragma unroll
            for (int u = 0; u < L::NU; ++u) r.y[k][u] = r.x[k][u];
        }
    }
    // The sum over k runs in kParts independent accumulators per n-tile so that consecutive MMAs do not wait on each
    // other's result (a dependent MMA costs its full latency); they are added at the end.
    constexpr int kParts = 4;
    float cp[kParts][NT][4];
#pragma unroll
    for (int pt = 0; pt < kParts; ++pt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int j = 0; j < 4; ++j) cp[pt][nt][j] = 0.f;
    const uint2 *bf = reinterpret_cast<const uint2 *>(smem + L::kOffBf);
#pragma unroll
    for (int t = 2; t >= 0; --t)            // smallest terms first
#pragma unroll
        for (int ks = 0; ks < L::NKS; ++ks)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint2 b = lds_u2(bf + ((t * L::NKS + ks) * NT + nt) * 32 + lane);
                mma16816(cp[ks % kParts][nt], r.y[0][2 * ks], r.y[1][2 * ks], r.y[0][2 * ks + 1], r.y[1][2 * ks + 1], b.x, b.y);
            }
    float c[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) c[nt][j] = (cp[0][nt][j] + cp[1][nt][j]) + (cp[2][nt][j] + cp[3][nt][j]);
    float d0 = 0.f, d1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int e = nt * 8 + 2 * q + (j & 1);
            const float s = e < a.E ? __fdividef(1.f, 1.f + __expf(-c[nt][j])) : 0.f;
            r.sg[nt][j] = s;
            if (j < 2) d0 += s; else d1 += s;
        }
    r.D[0] = fmaxf(quad_sum(d0), 1e-20f);
    r.D[1] = fmaxf(quad_sum(d1), 1e-20f);
}

template <int DH, int NT>
__device__ __forceinline__ void mma_load_rows(uint32_t (&dst)[2][DH / 8], const __nv_bfloat16 *p0, const __nv_bfloat16 *p1,
                                              bool ok0, bool ok1, int q) {
#pragma unroll
    for (int i = 0; i < DH / 32; ++i) {
        const uint4 z = make_uint4(0u, 0u, 0u, 0u);
        const uint4 v0 = ok0 ? __ldg(reinterpret_cast<const uint4 *>(p0) + i * 4 + q) : z;
        const uint4 v1 = ok1 ? __ldg(reinterpret_cast<const uint4 *>(p1) + i * 4 + q) : z;
        dst[0][4 * i] = v0.x; dst[0][4 * i + 1] = v0.y; dst[0][4 * i + 2] = v0.z; dst[0][4 * i + 3] = v0.w;
        dst[1][4 * i] = v1.x; dst[1][4 * i + 1] = v1.y; dst[1][4 * i + 2] = v1.z; dst[1][4 * i + 3] = v1.w;
    }
}
template <int DH>
__device__ __forceinline__ void mma_store_row(__nv_bfloat16 *p, const uint32_t (&v)[DH / 8], int q) {
#pragma unroll
    for (int i = 0; i < DH / 32; ++i)
        reinterpret_cast<uint4 *>(p)[i * 4 + q] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
}

// 16-token tile index dealt round-robin over warps, then block columns
__device__ __forceinline__ long long mma_tile_row(int it, int by, int gy, int warp) {
    return 16LL * (((long long)it * gy + by) * kWarps + warp);
}

template <int DH, int NT, bool NORM>
__global__ void __launch_bounds__(kWarps * 32, 2)
prologue_fwd_mma_kernel(const ProArgs a, __nv_bfloat16 *Q, float *R) {
    using L = MmaLayout<DH, NT>;
    extern __shared__ __align__(16) uint8_t smem_mma[];
    const int h = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
    build_router_fragments<DH, NT, false>(a.router + (long long)h * DH * a.E, a.E, smem_mma);
    float *wsm = reinterpret_cast<float *>(smem_mma + L::kOffW);
    for (int i = threadIdx.x; i < DH; i += blockDim.x) wsm[i] = NORM ? a.W[h * DH + i] : 1.f;
    __syncthreads();
    for (int it = 0;; ++it) {
        const long long t0 = mma_tile_row(it, blockIdx.y, gridDim.y, warp);
        if (t0 >= a.T) break;
        const long long tr[2] = {t0 + g, t0 + g + 8};
        const bool ok[2] = {tr[0] < a.T, tr[1] < a.T};
        MmaRows<DH, NT> r;
        mma_load_rows<DH, NT>(r.x, a.X + tr[0] * a.x_tok + h * DH, a.X + tr[1] * a.x_tok + h * DH, ok[0], ok[1], q);
        mma_rows_forward<DH, NT, NORM>(r, a, smem_mma, lane);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            if (!ok[k]) continue;
            if (NORM) mma_store_row<DH>(Q + tr[k] * a.x_tok + h * DH, r.y[k], q);
            const long long b = div_by_s(tr[k], a), s = tr[k] - b * a.S;
            float *rrow = R + ((b * a.H + h) * a.S + s) * a.E;
            const float inv = __fdividef(1.f, r.D[k]);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int e = nt * 8 + 2 * q + j;
                    if (e < a.E) rrow[e] = r.sg[nt][2 * k + j] * inv;
                }
        }
    }
}

template <int DH, int NT, bool NORM>
__global__ void __launch_bounds__(kWarps * 32, 1)
prologue_bwd_mma_kernel(const ProArgs a, const ProBwdArgs gp) {
    using L = MmaLayout<DH, NT>;
    constexpr int NU = L::NU, NMT = DH / 16;
    extern __shared__ __align__(16) uint8_t smem_mma[];
    const int h = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
    const int E = a.E, DE = DH * E;
    build_router_fragments<DH, NT, true>(a.router + (long long)h * DE, E, smem_mma);
    float *wsm = reinterpret_cast<float *>(smem_mma + L::kOffW);
    for (int i = threadIdx.x; i < DH; i += blockDim.x) wsm[i] = NORM ? a.W[h * DH + i] : 1.f;
    __syncthreads();
    const uint2 *b2 = reinterpret_cast<const uint2 *>(smem_mma + L::kOffB2f);

    float racc[NMT][NT][4];   // d router: 16 (permuted) rows d per mt, sub-networks nt*8 + 2q + {0,1}
    // d norm weight of this lane's columns (summed over its rows): private slots in shared memory, registers are short
    float *wacc = reinterpret_cast<float *>(smem_mma + L::kOffWacc + warp * L::kWacc) + lane;
#pragma unroll
    for (int mt = 0; mt < NMT; ++mt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int j = 0; j < 4; ++j) racc[mt][nt][j] = 0.f;
#pragma unroll
    for (int u = 0; u < 2 * NU; ++u) wacc[u * 32] = 0.f;

    // The next tile's X and dQ rows are copied into shared memory (cp.async, whole 256-byte rows per half-warp) while the
    // current tile is worked on; the warp then reads them in its fragment layout, X again for each use instead of keeping it.
    const uint32_t stage0 = smem_u32(smem_mma + L::kOffStage + warp * 2 * L::kStage);
    auto prefetch = [&](long long t0, int buf) {
        const uint32_t dst = stage0 + buf * L::kStage;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int row = 2 * j + (lane >> 4), cc = lane & 15;      // 16 chunks per row (d_h = 128); fewer for smaller d_h
            if (cc * 8 < DH) {
                const long long t = t0 + row;
                const bool okr = t < a.T;
                const long long b = okr ? div_by_s(t, a) : 0, sq = okr ? t - b * a.S : 0;
                const __nv_bfloat16 *xs = okr ? a.X + t * a.x_tok + h * DH + cc * 8 : a.X;
                const __nv_bfloat16 *qs = okr ? gp.dQ + b * gp.dq_b + (long long)h * gp.dq_h + sq * gp.dq_s + cc * 8 : gp.dQ;
                cp_async16(dst + row * L::kSRow + cc * 16, xs, okr);
                cp_async16(dst + L::kSTile + row * L::kSRow + cc * 16, qs, okr);
            }
        }
        cp_async_commit();
    };
    {
        const long long t_first = mma_tile_row(0, blockIdx.y, gridDim.y, warp);
        if (t_first < a.T) prefetch(t_first, 0);
    }

    for (int it = 0;; ++it) {
        const long long t0 = mma_tile_row(it, blockIdx.y, gridDim.y, warp);
        if (t0 >= a.T) break;
        const long long tnext = mma_tile_row(it + 1, blockIdx.y, gridDim.y, warp);
        if (tnext < a.T) {
            prefetch(tnext, (it + 1) & 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncwarp();
        const uint32_t xs = stage0 + (it & 1) * L::kStage, qs = xs + L::kSTile;
        const long long tr[2] = {t0 + g, t0 + g + 8};
        const bool ok[2] = {tr[0] < a.T, tr[1] < a.T};
        float ge[NT][4];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const long long b = ok[k] ? div_by_s(tr[k], a) : 0, sq = ok[k] ? tr[k] - b * a.S : 0;
            const float *rrow = gp.dR + ((b * a.H + h) * a.S + sq) * E;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int e = nt * 8 + 2 * q + j;
                    ge[nt][2 * k + j] = (ok[k] && e < E) ? __ldg(rrow + e) : 0.f;
                }
        }
        // 32-bit registers 4i..4i+3 of row g + 8k of a staged tile (the chunk 4i+q of that row)
        auto chunk = [&](uint32_t tile, int k, int i) { return lds_u4(tile + (g + 8 * k) * L::kSRow + (i * 4 + q) * 16); };
        MmaRows<DH, NT> r;
#pragma unroll
        for (int k = 0; k < 2; ++k)
#pragma unroll
            for (int i = 0; i < L::NI; ++i) {
                const uint4 v = chunk(xs, k, i);
                r.x[k][4 * i] = v.x; r.x[k][4 * i + 1] = v.y; r.x[k][4 * i + 2] = v.z; r.x[k][4 * i + 3] = v.w;
            }
        mma_rows_forward<DH, NT, NORM>(r, a, smem_mma, lane);

        // R_e = sg_e / D -> dsg_e = (g_e - sum_k g_k R_k) / D ; dlogit_e = dsg_e sg_e (1 - sg_e); a clamped D passes no gradient
        float inv[2], gr[2] = {0.f, 0.f};
#pragma unroll
        for (int k = 0; k < 2; ++k) inv[k] = __fdividef(1.f, r.D[k]);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int j = 0; j < 4; ++j) gr[j >> 1] = fmaf(ge[nt][j], r.sg[nt][j] * inv[j >> 1], gr[j >> 1]);
#pragma unroll
        for (int k = 0; k < 2; ++k) gr[k] = r.D[k] > 1e-20f ? quad_sum(gr[k]) : 0.f;
        uint32_t dlh[NT][2], dlm[NT][2], dll[NT][2];   // bf16 pairs of the hi, mid and lo terms: [nt][row]
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                float hi[2], mid[2], lo[2];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const float s = r.sg[nt][2 * k + j];
                    const float dl = (ge[nt][2 * k + j] - gr[k]) * inv[k] * s * (1.f - s);
                    split3(dl, hi[j], mid[j], lo[j]);
                }
                dlh[nt][k] = pack_bf16(hi[0], hi[1]);
                dlm[nt][k] = pack_bf16(mid[0], mid[1]);
                dll[nt][k] = pack_bf16(lo[0], lo[1]);
            }

        // d router += y^T dlogits : 16 x 8 tiles over d (m) and sub-networks (n), k = the 16 tokens.  Both operands are
        // transposed register fragments.  Rows of m-tile mt are the columns of y registers 2mt (m = 0..7) and 2mt+1
        // (m = 8..15): row m stands for d = mma_col(m >> 1, u) + (m & 1).
        {
            uint32_t bfr[3][NT][2];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                    bfr[0][nt][k] = movmatrix_trans(dlh[nt][k]);
                    bfr[1][nt][k] = movmatrix_trans(dlm[nt][k]);
                    bfr[2][nt][k] = movmatrix_trans(dll[nt][k]);
                }
            constexpr int MG = NMT % 4 == 0 ? 4 : 2;    // m-tiles per group (d_h = 96 has six)
#pragma unroll
            for (int m0 = 0; m0 < NMT; m0 += MG) {      // a group of m-tiles at a time, term by term: consecutive MMAs are independent
                uint32_t av[MG][4];
#pragma unroll
                for (int mm = 0; mm < MG; ++mm) {
                    const int mt = m0 + mm;
                    av[mm][0] = movmatrix_trans(r.y[0][2 * mt]);
                    av[mm][1] = movmatrix_trans(r.y[0][2 * mt + 1]);
                    av[mm][2] = movmatrix_trans(r.y[1][2 * mt]);
                    av[mm][3] = movmatrix_trans(r.y[1][2 * mt + 1]);
                }
#pragma unroll
                for (int t = 2; t >= 0; --t)
#pragma unroll
                    for (int mm = 0; mm < MG; ++mm)
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt)
                            mma16816(racc[m0 + mm][nt], av[mm][0], av[mm][1], av[mm][2], av[mm][3], bfr[t][nt][0], bfr[t][nt][1]);
            }
        }

        // dy = dQ + dlogits . router^T, n-tile u at a time (its accumulator columns are this lane's own columns
        // mma_col(q,u)+{0,1}); evaluated twice, once for the row sums RMSNorm's backward needs and once for dx, which
        // is cheaper than keeping d_h/2 accumulators alive.
        auto word = [](const uint4 &v, int m) { return m == 0 ? v.x : m == 1 ? v.y : m == 2 ? v.z : v.w; };
        auto dy_chunk = [&](int i, const uint4 &q0, const uint4 &q1, float (&dy)[4][4]) {   // n-tiles 4i .. 4i+3, term by term
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                dy[m][0] = bf16_lo(word(q0, m)); dy[m][1] = bf16_hi(word(q0, m));
                dy[m][2] = bf16_lo(word(q1, m)); dy[m][3] = bf16_hi(word(q1, m));
            }
#pragma unroll
            for (int kk = 0; kk < L::NKK; ++kk) {
                const bool two = 2 * kk + 1 < NT;
                const int n1 = two ? 2 * kk + 1 : 0;
                uint2 bh[4], bm[4];
#pragma unroll
                for (int m = 0; m < 4; ++m) {
                    bh[m] = lds_u2(b2 + ((0 * L::NKK + kk) * NU + 4 * i + m) * 32 + lane);
                    bm[m] = lds_u2(b2 + ((1 * L::NKK + kk) * NU + 4 * i + m) * 32 + lane);
                }
#pragma unroll
                for (int m = 0; m < 4; ++m)
                    mma16816(dy[m], dlm[2 * kk][0], dlm[2 * kk][1], two ? dlm[n1][0] : 0u, two ? dlm[n1][1] : 0u, bh[m].x, bh[m].y);
#pragma unroll
                for (int m = 0; m < 4; ++m)
                    mma16816(dy[m], dlh[2 * kk][0], dlh[2 * kk][1], two ? dlh[n1][0] : 0u, two ? dlh[n1][1] : 0u, bm[m].x, bm[m].y);
#pragma unroll
                for (int m = 0; m < 4; ++m)
                    mma16816(dy[m], dlh[2 * kk][0], dlh[2 * kk][1], two ? dlh[n1][0] : 0u, two ? dlh[n1][1] : 0u, bh[m].x, bh[m].y);
            }
        };

        // RMSNorm backward: y_d = w_d x_d rstd ; dx_d = rstd w_d dy_d - rstd^3 x_d mean_k(w_k dy_k x_k) ; dw_d += dy_d x_d rstd
        float r3c[2] = {0.f, 0.f};
        if (NORM) {
            float c[2] = {0.f, 0.f};
#pragma unroll
            for (int i = 0; i < L::NI; ++i) {
                const uint4 x0 = chunk(xs, 0, i), x1 = chunk(xs, 1, i), q0 = chunk(qs, 0, i), q1 = chunk(qs, 1, i);
                float dy4[4][4];
                dy_chunk(i, q0, q1, dy4);
#pragma unroll
                for (int m = 0; m < 4; ++m) {
                    const int u = 4 * i + m;
                    const float(&dy)[4] = dy4[m];
                    const float2 w = lds_f2(wsm + mma_col(q, u));
                    const uint32_t xw[2] = {word(x0, m), word(x1, m)};
                    float a0 = wacc[(2 * u) * 32], a1 = wacc[(2 * u + 1) * 32];
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        const float p0 = dy[2 * k] * bf16_lo(xw[k]), p1 = dy[2 * k + 1] * bf16_hi(xw[k]);
                        c[k] = fmaf(w.x, p0, fmaf(w.y, p1, c[k]));
                        a0 = fmaf(p0, r.rstd[k], a0);
                        a1 = fmaf(p1, r.rstd[k], a1);
                    }
                    wacc[(2 * u) * 32] = a0;
                    wacc[(2 * u + 1) * 32] = a1;
                }
            }
#pragma unroll
            for (int k = 0; k < 2; ++k) r3c[k] = r.rstd[k] * r.rstd[k] * r.rstd[k] * quad_sum(c[k]) * (1.f / (float)DH);
        }
#pragma unroll
        for (int i = 0; i < L::NI; ++i) {      // one 16-byte chunk of both rows at a time, stored as soon as it is complete
            const uint4 x0 = chunk(xs, 0, i), x1 = chunk(xs, 1, i), q0 = chunk(qs, 0, i), q1 = chunk(qs, 1, i);
            uint32_t dx[2][4];
            float dy4[4][4];
            dy_chunk(i, q0, q1, dy4);
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                const int u = 4 * i + m;
                const float(&dy)[4] = dy4[m];
                if (NORM) {
                    const float2 w = lds_f2(wsm + mma_col(q, u));
                    const uint32_t xw[2] = {word(x0, m), word(x1, m)};
#pragma unroll
                    for (int k = 0; k < 2; ++k)
                        dx[k][m] = pack_bf16(r.rstd[k] * w.x * dy[2 * k] - r3c[k] * bf16_lo(xw[k]),
                                             r.rstd[k] * w.y * dy[2 * k + 1] - r3c[k] * bf16_hi(xw[k]));
                } else {
#pragma unroll
                    for (int k = 0; k < 2; ++k) dx[k][m] = pack_bf16(dy[2 * k], dy[2 * k + 1]);
                }
            }
#pragma unroll
            for (int k = 0; k < 2; ++k)
                if (ok[k])
                    reinterpret_cast<uint4 *>(gp.dX + tr[k] * a.x_tok + h * DH)[i * 4 + q] =
                        make_uint4(dx[k][0], dx[k][1], dx[k][2], dx[k][3]);
        }
        __syncwarp();   // every lane is done with this stage before the copy of the tile after next overwrites it
    }

    // warps' accumulators -> shared -> this block's partial sums (fixed order).  The fragments are no longer
    // needed: the per-warp sums reuse shared memory from the start.
    float wsum[NU][2];
#pragma unroll
    for (int u = 0; u < NU; ++u) {
        wsum[u][0] = NORM ? wacc[(2 * u) * 32] : 0.f;
        wsum[u][1] = NORM ? wacc[(2 * u + 1) * 32] : 0.f;
    }
    __syncthreads();
    float *acc_r = reinterpret_cast<float *>(smem_mma), *acc_w = acc_r + kWarps * DE;
    float *my_r = acc_r + warp * DE, *my_w = acc_w + warp * DH;
#pragma unroll
    for (int mt = 0; mt < NMT; ++mt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int j = 0; j < 4; ++j) {   // accumulator row m = g (+8): see the d router product above
                const int d = mma_col(g >> 1, 2 * mt + (j >> 1)) + (g & 1), e = nt * 8 + 2 * q + (j & 1);
                if (e < E) my_r[d * E + e] = racc[mt][nt][j];
            }
#pragma unroll
    for (int u = 0; u < NU; ++u)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            float v = wsum[u][j];   // sum over the 8 lanes that hold the same columns
            v += __shfl_xor_sync(0xffffffffu, v, 4);
            v += __shfl_xor_sync(0xffffffffu, v, 8);
            v += __shfl_xor_sync(0xffffffffu, v, 16);
            if (g == 0) my_w[mma_col(q, u) + j] = v;
        }
    __syncthreads();
    for (int i = threadIdx.x; i < DE; i += blockDim.x) {
        float v = 0.f;
#pragma unroll
        for (int wp = 0; wp < kWarps; ++wp) v += acc_r[wp * DE + i];
        gp.part_router[((long long)blockIdx.y * a.H + h) * DE + i] = v;
    }
    if (NORM)
        for (int i = threadIdx.x; i < DH; i += blockDim.x) {
            float v = 0.f;
#pragma unroll
            for (int wp = 0; wp < kWarps; ++wp) v += acc_w[wp * DH + i];
            gp.part_w[((long long)blockIdx.y * a.H + h) * DH + i] = v;
        }
}

template <int DH, int NT>
size_t mma_fwd_smem() { return (size_t)MmaLayout<DH, NT>::kOffFwdEnd; }
template <int DH, int NT>
size_t mma_bwd_smem(int E) {
    const size_t loop = (size_t)MmaLayout<DH, NT>::kOffBwdEnd, fin = (size_t)kWarps * ((size_t)DH * E + DH) * sizeof(float);
    return loop > fin ? loop : fin;
}

template <int DH, int NT, bool NORM>
cudaError_t launch_fwd_mma(const ProArgs &a, dim3 grid, __nv_bfloat16 *Q, float *R, cudaStream_t st) {
    const size_t smem = mma_fwd_smem<DH, NT>();
    cudaError_t e = cudaFuncSetAttribute(prologue_fwd_mma_kernel<DH, NT, NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    prologue_fwd_mma_kernel<DH, NT, NORM><<<grid, kWarps * 32, smem, st>>>(a, Q, R);
    return cudaGetLastError();
}
template <int DH, int NT, bool NORM>
cudaError_t launch_bwd_mma(const ProArgs &a, dim3 grid, const ProBwdArgs &g, cudaStream_t st) {
    const size_t smem = mma_bwd_smem<DH, NT>(a.E);
    cudaError_t e = cudaFuncSetAttribute(prologue_bwd_mma_kernel<DH, NT, NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    prologue_bwd_mma_kernel<DH, NT, NORM><<<grid, kWarps * 32, smem, st>>>(a, g);
    return cudaGetLastError();
}
