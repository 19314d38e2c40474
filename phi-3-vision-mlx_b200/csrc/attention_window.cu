// Paged attention over a ragged batch with a sliding window, a per-head sink in the softmax denominator and a per-head distance
// penalty: score(i, j) = scale * q_i . k_j - pen[h][i - j], visible when 0 <= i - j < window (window 0: every earlier key),
// weights = exp(score) / (exp(sink_h) + sum over visible exp(score)); optional per-(token, head) output gate. Head sizes of
// keys (dim) and values (vdim) are independent run-time numbers (<= 256), grouped-query heads share K/V (head h reads h / (H/G)).
//
// All keys come from the page pools ([page][kv head][64 tokens][dim | vdim], fp32 or bf16): the caller writes the step's own K/V
// first. Scores, softmax and the P.V sums are fp32 on the FMA pipes in both storage modes, which is what the all-fp32 serving mode
// needs; the sink is folded in as the INITIAL state of the online softmax (running max = sink, denominator = 1, no value).
//   attn_window_prefill_kernel: one CTA = 32 consecutive query tokens of one sequence x one head, key tiles = whole pages, only
//                               the pages that hold a visible key are visited
//   attn_window_decode_kernel:  one CTA = one single-token request x one K/V head (all of its query heads share the K/V reads),
//                               warps stride over the visible keys, partial softmax states merged through shared memory
#include "common.cuh"
#include "../../include/phi3_b200.h"
#include <cfloat>

namespace {
template <typename T> __device__ __forceinline__ float ldv(const T* p);
template <> __device__ __forceinline__ float ldv<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldv<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stv(T* p, float v);
template <> __device__ __forceinline__ void stv<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stv<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

constexpr int BQ = 32, WARPS = 4, RPW = BQ / WARPS;          // prefill: query rows per CTA / per warp

template <typename AT, typename CT, int DVC>
__global__ void __launch_bounds__(WARPS * 32) attn_window_prefill_kernel(p3_attn_window_args a) {
    extern __shared__ __align__(16) float sm[];
    const int d = a.dim, dv = a.vdim, dp = (d + 3) & ~3;       // q rows padded to float4
    float* Qs = sm;                                          // [BQ][dp]
    float* Ks = Qs + BQ * dp;                                // [64][dp + 1]
    float* Vs = Ks + P3_PAGE * (dp + 1);                     // [64][dv]
    float* Ss = Vs + P3_PAGE * dv;                           // [BQ][64 + 4]
    const int4 tile = reinterpret_cast<const int4*>(a.tiles)[blockIdx.x];
    const int row0 = tile.x, nq = tile.y, slot = tile.z, pos0 = tile.w;
    const int h = blockIdx.y, g = h / (a.n_heads / a.n_kv);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const AT* q = (const AT*)a.q;
    for (int i = tid; i < BQ * dp; i += blockDim.x) {
        const int r = i / dp, c = i % dp;
        Qs[i] = (r < nq && c < d) ? ldv(q + (size_t)(row0 + r) * a.ld_q + (size_t)h * d + c) * a.scale : 0.f;
    }
    const float sink = a.sink ? a.sink[h] : -FLT_MAX;
    float m[RPW], l[RPW], acc[RPW][DVC];
#pragma unroll
    for (int r = 0; r < RPW; r++) {
        m[r] = sink; l[r] = a.sink ? 1.f : 0.f;
#pragma unroll
        for (int j = 0; j < DVC; j++) acc[r][j] = 0.f;
    }
    const int last = pos0 + nq - 1;
    const int first = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
    const int32_t* bt = a.block_table + (size_t)slot * a.bt_stride;
    const float* pen = a.penalty ? a.penalty + (size_t)h * a.n_penalty : nullptr;
    for (int pg = first / P3_PAGE; pg <= last / P3_PAGE; pg++) {
        const int page = bt[pg];
        const CT* kp = (const CT*)a.k_pool + ((size_t)page * a.n_kv + g) * P3_PAGE * d;
        const CT* vp = (const CT*)a.v_pool + ((size_t)page * a.n_kv + g) * P3_PAGE * dv;
        __syncthreads();                                     // previous tile fully consumed (and Qs written, first time)
        for (int i = tid; i < P3_PAGE * d; i += blockDim.x) Ks[(i / d) * (dp + 1) + (i % d)] = ldv(kp + i);
        for (int i = tid; i < P3_PAGE * dv; i += blockDim.x) Vs[i] = ldv(vp + i);
        __syncthreads();
        // scores: this warp's RPW rows x keys (lane, lane + 32)
        float s[RPW][2];
#pragma unroll
        for (int r = 0; r < RPW; r++) s[r][0] = s[r][1] = 0.f;
        const float* k0 = Ks + lane * (dp + 1);
        const float* k1 = Ks + (lane + 32) * (dp + 1);
        for (int i = 0; i < d; i += 4) {
            float ka[4], kb[4];
#pragma unroll
            for (int e = 0; e < 4; e++) { const bool in = i + e < d; ka[e] = in ? k0[i + e] : 0.f; kb[e] = in ? k1[i + e] : 0.f; }
#pragma unroll
            for (int r = 0; r < RPW; r++) {
                const float4 qv = *reinterpret_cast<const float4*>(Qs + (warp * RPW + r) * dp + i);
                s[r][0] = fmaf(qv.x, ka[0], s[r][0]); s[r][0] = fmaf(qv.y, ka[1], s[r][0]);
                s[r][0] = fmaf(qv.z, ka[2], s[r][0]); s[r][0] = fmaf(qv.w, ka[3], s[r][0]);
                s[r][1] = fmaf(qv.x, kb[0], s[r][1]); s[r][1] = fmaf(qv.y, kb[1], s[r][1]);
                s[r][1] = fmaf(qv.z, kb[2], s[r][1]); s[r][1] = fmaf(qv.w, kb[3], s[r][1]);
            }
        }
        // mask, penalty, online softmax; P goes to shared memory for the P.V pass
#pragma unroll
        for (int r = 0; r < RPW; r++) {
            const int qr = warp * RPW + r, qpos = pos0 + qr;
            float pv[2];
            float tmax = -FLT_MAX;
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int kpos = pg * P3_PAGE + lane + 32 * e, dist = qpos - kpos;
                const bool vis = qr < nq && dist >= 0 && (a.window <= 0 || dist < a.window);
                float v = -FLT_MAX;
                if (vis) v = s[r][e] - (pen ? pen[min(dist, a.n_penalty - 1)] : 0.f);
                pv[e] = v;
                tmax = fmaxf(tmax, v);
            }
            tmax = warp_max(tmax);
            const float mn = fmaxf(m[r], tmax);
            const float corr = expf(m[r] - mn);               // m is finite (sink) or -FLT_MAX; both give a finite difference or 0
            float ps = 0.f;
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const float p = pv[e] > -FLT_MAX ? expf(pv[e] - mn) : 0.f;
                Ss[qr * (P3_PAGE + 4) + lane + 32 * e] = p;
                ps += p;
            }
            ps = warp_sum(ps);
            l[r] = l[r] * corr + ps;
            m[r] = mn;
#pragma unroll
            for (int j = 0; j < DVC; j++) acc[r][j] *= corr;
        }
        __syncwarp();
        // P.V: lane owns value columns lane + 32 j
        for (int k = 0; k < P3_PAGE; k += 4) {
            float vv[4][DVC];
#pragma unroll
            for (int e = 0; e < 4; e++)
#pragma unroll
                for (int j = 0; j < DVC; j++) { const int c = lane + 32 * j; vv[e][j] = c < dv ? Vs[(k + e) * dv + c] : 0.f; }
#pragma unroll
            for (int r = 0; r < RPW; r++) {
                const float4 p = *reinterpret_cast<const float4*>(Ss + (warp * RPW + r) * (P3_PAGE + 4) + k);
#pragma unroll
                for (int j = 0; j < DVC; j++) {
                    acc[r][j] = fmaf(p.x, vv[0][j], acc[r][j]); acc[r][j] = fmaf(p.y, vv[1][j], acc[r][j]);
                    acc[r][j] = fmaf(p.z, vv[2][j], acc[r][j]); acc[r][j] = fmaf(p.w, vv[3][j], acc[r][j]);
                }
            }
        }
    }
    AT* out = (AT*)a.out;
#pragma unroll
    for (int r = 0; r < RPW; r++) {
        const int qr = warp * RPW + r;
        if (qr >= nq) continue;
        const float gate = a.gate ? a.gate[(size_t)(row0 + qr) * a.n_heads + h] : 1.f;
        const float inv = l[r] > 0.f ? gate / l[r] : 0.f;
#pragma unroll
        for (int j = 0; j < DVC; j++) {
            const int c = lane + 32 * j;
            if (c < dv) stv(out + (size_t)(row0 + qr) * a.ld_out + (size_t)h * dv + c, acc[r][j] * inv);
        }
    }
}

constexpr int DW = 4, RMAX = 8;                              // decode: warps per CTA, query heads per pass

template <typename AT, typename CT, int DC, int DVC>
__global__ void __launch_bounds__(DW * 32) attn_window_decode_kernel(p3_attn_window_args a) {
    extern __shared__ __align__(16) float sm[];
    const int d = a.dim, dv = a.vdim, rep = a.n_heads / a.n_kv;
    float* Qs = sm;                                          // [RMAX][d]
    float* Ms = Qs + RMAX * d;                               // [DW][RMAX]
    float* Ls = Ms + DW * RMAX;                              // [DW][RMAX]
    float* As = Ls + DW * RMAX;                              // [DW][RMAX][dv]
    const int4 tile = reinterpret_cast<const int4*>(a.tiles)[blockIdx.x];
    const int row = tile.x, slot = tile.z, pos = tile.w;
    const int g = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int first = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    const int32_t* bt = a.block_table + (size_t)slot * a.bt_stride;
    const AT* q = (const AT*)a.q + (size_t)row * a.ld_q;
    AT* out = (AT*)a.out + (size_t)row * a.ld_out;
    for (int h0 = 0; h0 < rep; h0 += RMAX) {
        const int nr = min(RMAX, rep - h0), hb = g * rep + h0;
        __syncthreads();
        for (int i = tid; i < nr * d; i += blockDim.x) Qs[i] = ldv(q + (size_t)hb * d + i) * a.scale;
        __syncthreads();
        float m[RMAX], l[RMAX], acc[RMAX][DVC];
#pragma unroll
        for (int r = 0; r < RMAX; r++) {
            const bool s0 = warp == 0 && a.sink && r < nr;   // the sink enters once: as warp 0's initial state
            m[r] = s0 ? a.sink[hb + r] : -FLT_MAX; l[r] = s0 ? 1.f : 0.f;
#pragma unroll
            for (int j = 0; j < DVC; j++) acc[r][j] = 0.f;
        }
        for (int kpos = first + warp; kpos <= pos; kpos += DW) {
            const int page = bt[kpos / P3_PAGE], off = kpos % P3_PAGE;
            const CT* kp = (const CT*)a.k_pool + (((size_t)page * a.n_kv + g) * P3_PAGE + off) * d;
            const CT* vp = (const CT*)a.v_pool + (((size_t)page * a.n_kv + g) * P3_PAGE + off) * dv;
            float kr[DC], vr[DVC];
#pragma unroll
            for (int j = 0; j < DC; j++) { const int c = lane + 32 * j; kr[j] = c < d ? ldv(kp + c) : 0.f; }
#pragma unroll
            for (int j = 0; j < DVC; j++) { const int c = lane + 32 * j; vr[j] = c < dv ? ldv(vp + c) : 0.f; }
            const int dist = pos - kpos;
#pragma unroll
            for (int r = 0; r < RMAX; r++) {
                if (r >= nr) break;
                float s = 0.f;
#pragma unroll
                for (int j = 0; j < DC; j++) { const int c = lane + 32 * j; if (c < d) s = fmaf(Qs[r * d + c], kr[j], s); }
                s = warp_sum(s);
                if (a.penalty) s -= a.penalty[(size_t)(hb + r) * a.n_penalty + min(dist, a.n_penalty - 1)];
                const float mn = fmaxf(m[r], s), corr = expf(m[r] - mn), p = expf(s - mn);
                l[r] = l[r] * corr + p;
                m[r] = mn;
#pragma unroll
                for (int j = 0; j < DVC; j++) acc[r][j] = fmaf(p, vr[j], acc[r][j] * corr);
            }
        }
        // merge the warps' partial states
#pragma unroll
        for (int r = 0; r < RMAX; r++) {
            if (r >= nr) break;
            if (lane == 0) { Ms[warp * RMAX + r] = m[r]; Ls[warp * RMAX + r] = l[r]; }
#pragma unroll
            for (int j = 0; j < DVC; j++) { const int c = lane + 32 * j; if (c < dv) As[(size_t)(warp * RMAX + r) * dv + c] = acc[r][j]; }
        }
        __syncthreads();
        for (int i = tid; i < nr * dv; i += blockDim.x) {
            const int r = i / dv, c = i % dv;
            float M = -FLT_MAX;
            for (int w = 0; w < DW; w++) M = fmaxf(M, Ms[w * RMAX + r]);
            float L = 0.f, o = 0.f;
            for (int w = 0; w < DW; w++) {
                const float f = Ls[w * RMAX + r] > 0.f ? expf(Ms[w * RMAX + r] - M) : 0.f;
                L = fmaf(Ls[w * RMAX + r], f, L);
                o = fmaf(As[(size_t)(w * RMAX + r) * dv + c], f, o);
            }
            const float gate = a.gate ? a.gate[(size_t)row * a.n_heads + hb + r] : 1.f;
            stv(out + (size_t)(hb + r) * dv + c, L > 0.f ? o * gate / L : 0.f);
        }
    }
}

int check_args(const p3_attn_window_args* a, const char* who) {
    P3_CHECK_ARG(a && a->q && a->k_pool && a->v_pool && a->block_table && a->out && a->tiles, "%s: null argument", who);
    P3_CHECK_ARG(a->n_heads >= 1 && a->n_kv >= 1 && a->n_heads % a->n_kv == 0, "%s: heads must be a multiple of kv heads", who);
    P3_CHECK_ARG(a->dim >= 1 && a->dim <= 256 && a->vdim >= 1 && a->vdim <= 256, "%s: head sizes must be in [1, 256]", who);
    P3_CHECK_ARG(!a->penalty || a->n_penalty >= 1, "%s: empty penalty table", who);
    P3_CHECK_ARG(a->act_f32 == a->cache_f32, "%s: activations and cache must both be fp32 or both bf16", who);
    return 0;
}

template <typename K>
int set_smem(K kernel, size_t bytes, const char* who) {
    if (bytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        P3_CHECK_ARG(e == cudaSuccess, "%s: shared memory attribute: %s", who, cudaGetErrorString(e));
    }
    return 0;
}

template <typename AT, typename CT>
int launch_prefill(const p3_attn_window_args* a, cudaStream_t st) {
    const int dp = (a->dim + 3) & ~3;
    const size_t bytes = sizeof(float) * ((size_t)BQ * dp + (size_t)P3_PAGE * (dp + 1) + (size_t)P3_PAGE * a->vdim + (size_t)BQ * (P3_PAGE + 4));
    const dim3 grid((unsigned)a->n_tiles, (unsigned)a->n_heads);
    const int c = (a->vdim + 31) / 32;
#define GO(N)                                                                                              \
    do { if (set_smem(attn_window_prefill_kernel<AT, CT, N>, bytes, "attn_window_prefill")) return -1;      \
         attn_window_prefill_kernel<AT, CT, N><<<grid, WARPS * 32, bytes, st>>>(*a); } while (0)
    if (c <= 1) GO(1); else if (c <= 2) GO(2); else if (c <= 4) GO(4); else GO(8);
#undef GO
    return 0;
}

template <typename AT, typename CT>
int launch_decode(const p3_attn_window_args* a, cudaStream_t st) {
    const size_t bytes = sizeof(float) * ((size_t)RMAX * a->dim + 2 * DW * RMAX + (size_t)DW * RMAX * a->vdim);
    const dim3 grid((unsigned)a->n_tiles, (unsigned)a->n_kv);
    const int c = (a->dim + 31) / 32, cv = (a->vdim + 31) / 32;
#define GO(N, NV)                                                                                          \
    do { if (set_smem(attn_window_decode_kernel<AT, CT, N, NV>, bytes, "attn_window_decode")) return -1;    \
         attn_window_decode_kernel<AT, CT, N, NV><<<grid, DW * 32, bytes, st>>>(*a); } while (0)
#define GOV(N) do { if (cv <= 1) GO(N, 1); else if (cv <= 2) GO(N, 2); else if (cv <= 4) GO(N, 4); else GO(N, 8); } while (0)
    if (c <= 1) GOV(1); else if (c <= 2) GOV(2); else if (c <= 4) GOV(4); else GOV(8);
#undef GOV
#undef GO
    return 0;
}
}  // namespace

extern "C" int p3_attn_window_prefill(const p3_attn_window_args* a, cudaStream_t st) {
    if (check_args(a, "attn_window_prefill")) return -1;
    if (a->n_tiles == 0) return 0;
    const int rc = a->act_f32 ? launch_prefill<float, float>(a, st) : launch_prefill<bf16, bf16>(a, st);
    if (rc) return rc;
    P3_CHECK_LAUNCH("attn_window_prefill");
    return 0;
}

extern "C" int p3_attn_window_decode(const p3_attn_window_args* a, cudaStream_t st) {
    if (check_args(a, "attn_window_decode")) return -1;
    if (a->n_tiles == 0) return 0;
    const int rc = a->act_f32 ? launch_decode<float, float>(a, st) : launch_decode<bf16, bf16>(a, st);
    if (rc) return rc;
    P3_CHECK_LAUNCH("attn_window_decode");
    return 0;
}
