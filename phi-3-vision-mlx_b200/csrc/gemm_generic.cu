// p3_gemm_any: out[M,N] = X[M,K] * W[N,K]^T (+ bias) for ANY sizes, strides and alignments, operands fp32 or bf16, fp32
// accumulation in ascending k (one FMA chain per output element, so a row's result does not depend on which other rows share
// the launch). Two extras make it the mixture-of-experts workhorse: the rows of X can be gathered through an index list, and
// the rows can be cut into segments that each multiply with their own weight matrix (device-side segment offsets, so the host
// never learns how many tokens an expert received). A launch can also hold a batch of independent products over column blocks of
// X and out (one per attention head), with an optional sigmoid gate on the result.
//
// fp32 operands run on the FMA pipes (this is the "true 32-bit" path: no TF32). bf16 operands of aligned shapes run on the
// tensor cores through mma.sync m16n8k16 (fp32 accumulators); the dense bf16 projections with K % 8 == 0 go to the tcgen05
// kernel (p3_gemm) instead — this file is what is left: grouped expert products, fp32, and shapes p3_gemm does not take.
#include "common.cuh"
#include "../../include/phi3_b200.h"

namespace {
constexpr int BM = 64, BN = 64, BK = 16;

struct AnyP {
    const void* X; int64_t ldx; const int32_t* x_rows; int x_row_div;
    const void* W; int64_t ldw; int64_t w_gstride;
    const float* bias; int64_t bias_gstride;
    void* out; int64_t ldo;
    int64_t M; int N, K;
    const int32_t* seg; int n_groups;
    // a batch of nb products over column blocks of X and out: blockIdx.x = m-tile * nb + product, so that the CTAs in flight
    // together read whole rows of X and write whole rows of out (neighbouring column blocks) instead of one narrow column each
    int nb; int64_t x_bs, w_bs, o_bs; const float* gate; int64_t ld_gate;
};

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return __ldg(p); }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// which (group, first row, end row) does m-tile `tile` cover? Groups are walked in order; a launch has at most
// ceil(M / BM) + n_groups tiles, surplus CTAs leave.
__device__ __forceinline__ bool find_tile(const AnyP& p, int tile, int& g, int64_t& m0, int64_t& m1) {
    if (!p.seg) { g = 0; m0 = (int64_t)tile * BM; m1 = p.M; return m0 < m1; }
    int t = tile;
    for (int e = 0; e < p.n_groups; e++) {
        const int a = p.seg[e], b = p.seg[e + 1], nt = (b - a + BM - 1) / BM;
        if (t < nt) { g = e; m0 = a + (int64_t)t * BM; m1 = b; return true; }
        t -= nt;
    }
    return false;
}

template <typename XT, typename WT, typename OT>
__global__ void __launch_bounds__(256) gemm_any_fma_kernel(AnyP p) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    __shared__ __align__(16) float As[BK][BM + 4];
    __shared__ __align__(16) float Bs[BK][BN + 4];
    int g; int64_t m0, m1;
    const int bz = blockIdx.x % p.nb;
    if (!find_tile(p, blockIdx.x / p.nb, g, m0, m1)) return;
    const int n0 = blockIdx.y * BN, tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const XT* X = (const XT*)p.X + (size_t)bz * p.x_bs;
    const WT* W = (const WT*)p.W + (size_t)g * p.w_gstride + (size_t)bz * p.w_bs;
    // this thread stages row (tid / 4) of each tile, k = (tid % 4) * 4 .. + 3
    const int lr = tid >> 2, lk = (tid & 3) * 4;
    const int64_t am = m0 + lr;
    const XT* arow = nullptr;
    if (am < m1) arow = X + (size_t)(p.x_rows ? p.x_rows[am] / p.x_row_div : am) * p.ldx;
    const WT* brow = (n0 + lr < p.N) ? W + (size_t)(n0 + lr) * p.ldw : nullptr;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < p.K; k0 += BK) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int k = k0 + lk + j;
            As[lk + j][lr] = (arow && k < p.K) ? ldf(arow + k) : 0.f;
            Bs[lk + j][lr] = (brow && k < p.K) ? ldf(brow + k) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; k++) {
            const float4 a = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
            const float4 b = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
    const float* bias = p.bias ? p.bias + (size_t)g * p.bias_gstride : nullptr;
    OT* out = (OT*)p.out + (size_t)bz * p.o_bs;
    const float* gate = p.gate ? p.gate + (size_t)bz * p.o_bs : nullptr;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int64_t m = m0 + ty * 4 + i;
        if (m >= m1) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n >= p.N) continue;
            float v = acc[i][j] + (bias ? bias[n] : 0.f);
            if (gate) v *= 1.0f / (1.0f + expf(-gate[(size_t)m * p.ld_gate + n]));
            stf(out + (size_t)m * p.ldo + n, v);
        }
    }
}

// bf16 x bf16 on the tensor cores: 64 x 64 tile, 4 warps (2 x 2), each warp 32 x 32 = 2 x 4 MMAs of m16n8k16 per 16-wide k
// step; operands staged through shared memory as bf16 (row-major [row][k], 16-byte chunks, K % 8 == 0 and 16-byte aligned rows
// required by the launcher). Same tile walk, gather and segment logic as the FMA kernel. A k-slab is 128 elements: 16 lanes read
// the 256 contiguous bytes of one row, so that with few rows, where the kernel is a stream of W, DRAM sees bursts instead of
// 64-byte pieces of 64 rows; the next slab's loads are in flight while this one is multiplied.
// TK = k elements per stage: 128, or 64 for products with K <= 64 (the per-head products of an attention mixer), which would
// otherwise multiply a half-empty slab and hold twice the staging registers.
template <typename OT, int TK>
__global__ void __launch_bounds__(128) gemm_any_mma_kernel(AnyP p) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    __shared__ __align__(16) bf16 As[BM][TK + 8];
    __shared__ __align__(16) bf16 Bs[BN][TK + 8];
    int g; int64_t m0, m1;
    const int bz = blockIdx.x % p.nb;
    if (!find_tile(p, blockIdx.x / p.nb, g, m0, m1)) return;
    const int n0 = blockIdx.y * BN, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;
    const bf16* X = (const bf16*)p.X + (size_t)bz * p.x_bs;
    const bf16* W = (const bf16*)p.W + (size_t)g * p.w_gstride + (size_t)bz * p.w_bs;
    // staging: 64 rows x TK / 8 chunks of 8 elements per operand; LPR lanes per row, RPR rows per round of the CTA, NR rounds;
    // round j: row RPR j + (32 / LPR) warp + lane / LPR, chunk lane % LPR
    constexpr int LPR = TK / 8, RPR = 128 / LPR, NR = BM / RPR;
    const int srow0 = (32 / LPR) * warp + lane / LPR, schunk = (lane % LPR) * 8;
    int64_t aoff[NR];                                       // element offset of this thread's A row in round j, -1: no such row
#pragma unroll
    for (int j = 0; j < NR; j++) {
        const int64_t am = m0 + srow0 + RPR * j;
        aoff[j] = (am < m1) ? (int64_t)(p.x_rows ? p.x_rows[am] / p.x_row_div : am) * p.ldx : -1;
    }
    const bf16* brow0 = W + (size_t)(n0 + srow0) * p.ldw;
    float acc[2][4][4] = {};
    const uint4 zero = make_uint4(0, 0, 0, 0);
    uint4 ra[NR], rb[NR];
    auto fetch = [&](int k0) {
        const int k = k0 + schunk;
        const bool in = k < p.K;                           // K % 8 == 0: a chunk is inside or outside as a whole
#pragma unroll
        for (int j = 0; j < NR; j++) {
            ra[j] = (aoff[j] >= 0 && in) ? __ldg(reinterpret_cast<const uint4*>(X + aoff[j] + k)) : zero;
            rb[j] = (n0 + srow0 + RPR * j < p.N && in) ? ldg_nc_v4(brow0 + (size_t)(RPR * j) * p.ldw + k) : zero;
        }
    };
    fetch(0);
    for (int k0 = 0; k0 < p.K; k0 += TK) {
#pragma unroll
        for (int j = 0; j < NR; j++) {
            *reinterpret_cast<uint4*>(&As[srow0 + RPR * j][schunk]) = ra[j];
            *reinterpret_cast<uint4*>(&Bs[srow0 + RPR * j][schunk]) = rb[j];
        }
        __syncthreads();
        if (k0 + TK < p.K) fetch(k0 + TK);
#pragma unroll
        for (int kk = 0; kk < TK; kk += 16) {
            uint32_t a[2][4], b[4][2];
#pragma unroll
            for (int i = 0; i < 2; i++) {
                const int r = wm + i * 16 + (lane >> 2), c = kk + (lane & 3) * 2;
                a[i][0] = *reinterpret_cast<const uint32_t*>(&As[r][c]);
                a[i][1] = *reinterpret_cast<const uint32_t*>(&As[r + 8][c]);
                a[i][2] = *reinterpret_cast<const uint32_t*>(&As[r][c + 8]);
                a[i][3] = *reinterpret_cast<const uint32_t*>(&As[r + 8][c + 8]);
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int r = wn + j * 8 + (lane >> 2), c = kk + (lane & 3) * 2;
                b[j][0] = *reinterpret_cast<const uint32_t*>(&Bs[r][c]);
                b[j][1] = *reinterpret_cast<const uint32_t*>(&Bs[r][c + 8]);
            }
#pragma unroll
            for (int i = 0; i < 2; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) mma_bf16_16816(acc[i][j], a[i], b[j][0], b[j][1]);
        }
        __syncthreads();
    }
    const float* bias = p.bias ? p.bias + (size_t)g * p.bias_gstride : nullptr;
    OT* out = (OT*)p.out + (size_t)bz * p.o_bs;
    const float* gate = p.gate ? p.gate + (size_t)bz * p.o_bs : nullptr;
    // a thread holds pairs of neighbouring columns: one 4- or 8-byte store per pair where the pair is aligned
    const bool pair_ok = (p.ldo % 2 == 0) && (p.o_bs % 2 == 0) && (((uintptr_t)p.out) % (2 * sizeof(OT)) == 0);
#pragma unroll
    for (int i = 0; i < 2; i++)
#pragma unroll
        for (int j = 0; j < 4; j++)
#pragma unroll
            for (int hlf = 0; hlf < 2; hlf++) {
                const int64_t m = m0 + wm + i * 16 + (lane >> 2) + hlf * 8;
                const int n = n0 + wn + j * 8 + (lane & 3) * 2;
                if (m >= m1 || n >= p.N) continue;
                float v0 = acc[i][j][hlf * 2] + (bias ? bias[n] : 0.f);
                float v1 = (n + 1 < p.N) ? acc[i][j][hlf * 2 + 1] + (bias ? bias[n + 1] : 0.f) : 0.f;
                if (gate) {
                    v0 *= 1.0f / (1.0f + expf(-gate[(size_t)m * p.ld_gate + n]));
                    if (n + 1 < p.N) v1 *= 1.0f / (1.0f + expf(-gate[(size_t)m * p.ld_gate + n + 1]));
                }
                OT* o = out + (size_t)m * p.ldo + n;
                if (pair_ok && n + 1 < p.N) {
                    if constexpr (sizeof(OT) == 4) *reinterpret_cast<float2*>(o) = make_float2(v0, v1);
                    else *reinterpret_cast<uint32_t*>(o) = pack_bf16(v0, v1);
                } else {
                    stf(o, v0);
                    if (n + 1 < p.N) stf(o + 1, v1);
                }
            }
}
}  // namespace

extern "C" int p3_gemm_any(const p3_gemm_any_args* a, cudaStream_t st) {
    P3_CHECK_ARG(a && a->X && a->W && a->out, "gemm_any: null operand");
    P3_CHECK_ARG(a->M >= 0 && a->N >= 1 && a->K >= 1 && a->M < (1ll << 30), "gemm_any: bad sizes");
    P3_CHECK_ARG(!a->seg_offsets || a->n_groups >= 1, "gemm_any: segments need n_groups >= 1");
    P3_CHECK_ARG(!a->x_rows || a->x_row_div >= 1, "gemm_any: gather needs x_row_div >= 1");
    P3_CHECK_ARG(a->x_f32 == a->w_f32, "gemm_any: X and W must have the same element type");
    if (a->M == 0) return 0;
    AnyP p{a->X, a->ldx, a->x_rows, a->x_row_div, a->W, a->ldw, a->w_group_stride, a->bias, a->bias_group_stride,
           a->out, a->ldo, a->M, a->N, a->K, a->seg_offsets, a->seg_offsets ? a->n_groups : 1,
           a->n_batch > 1 ? a->n_batch : 1, a->x_batch_stride, a->w_batch_stride, a->out_batch_stride, a->gate, a->ld_gate};
    const int nb = p.nb;
    P3_CHECK_ARG(nb <= 65535, "gemm_any: too many products in a batch");
    if (nb == 1) p.x_bs = p.w_bs = p.o_bs = 0;
    const unsigned mt = (unsigned)((a->M + BM - 1) / BM) + (a->seg_offsets ? (unsigned)a->n_groups : 0u);
    const dim3 grid(mt * (unsigned)nb, (unsigned)((a->N + BN - 1) / BN));
    if (a->x_f32) {
        if (a->out_f32) p3_launch_pdl(gemm_any_fma_kernel<float, float, float>, dim3(grid), dim3(256), (size_t)(0), st, p);
        else p3_launch_pdl(gemm_any_fma_kernel<float, float, bf16>, dim3(grid), dim3(256), (size_t)(0), st, p);
    } else {
        const bool tc = a->K % 8 == 0 && a->ldx % 8 == 0 && a->ldw % 8 == 0 && a->w_group_stride % 8 == 0 &&
                        (nb == 1 || (a->x_batch_stride % 8 == 0 && a->w_batch_stride % 8 == 0)) &&
                        ((uintptr_t)a->X & 15) == 0 && ((uintptr_t)a->W & 15) == 0 && !a->force_fma;
        if (tc) {
            if (a->K <= 64) {
                if (a->out_f32) p3_launch_pdl(gemm_any_mma_kernel<float, 64>, dim3(grid), dim3(128), (size_t)(0), st, p);
                else p3_launch_pdl(gemm_any_mma_kernel<bf16, 64>, dim3(grid), dim3(128), (size_t)(0), st, p);
            } else if (a->out_f32) p3_launch_pdl(gemm_any_mma_kernel<float, 128>, dim3(grid), dim3(128), (size_t)(0), st, p);
            else p3_launch_pdl(gemm_any_mma_kernel<bf16, 128>, dim3(grid), dim3(128), (size_t)(0), st, p);
        } else {
            if (a->out_f32) p3_launch_pdl(gemm_any_fma_kernel<bf16, bf16, float>, dim3(grid), dim3(256), (size_t)(0), st, p);
            else p3_launch_pdl(gemm_any_fma_kernel<bf16, bf16, bf16>, dim3(grid), dim3(256), (size_t)(0), st, p);
        }
    }
    P3_CHECK_LAUNCH("gemm_any");
    return 0;
}
