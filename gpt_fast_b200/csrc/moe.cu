// Mixture of experts: a router that picks `top` of E small gated feed-forwards per token, and the experts.
//
// gfb_moe_router        few tokens: router logits and choice in one launch (a block per token)
// gfb_moe_route         from 32-bit router logits: s = sigmoid(z); the `top` experts with the largest s + correction
//                       (lowest index on ties); weights s / (sum of the chosen s + 1e-20) * scale.  Or (mode ROUTE_SOFTMAX_TOP)
//                       the `top` largest logits themselves, weighted by the softmax over just those, times scale
// gfb_moe_glu           act[pair, f] = g * sigmoid(alpha g) * (u + shift),  g = min(gate_f . h, limit),
//                       u = clamp(up_f . h, -limit, limit), for every (token, chosen expert) pair
// gfb_moe_down          x[t] += sum over the token's chosen experts of weight * (W_down act[pair]); 32-bit sum into the stream
//
// The gate and up rows of an expert alternate in one matrix w13 [E, 2F, D], the down matrix is w2 [E, D, F].
// A pair is p = t * top + r (r: rank of the expert among the token's choices).
//
// Two forms of the expert products.  Few tokens (a decode step): a warp per output number streams the weight row once,
// 16 bytes per lane and load, the token's input staged in shared memory.  Many tokens (a prompt): the pairs are sorted by
// expert (gfb_moe_plan: each expert's rows padded to whole tiles) and the products run tile by tile, each tile with its
// expert's weights, the rows' results brought back to pair order.  The tiles run on the tensor cores (bfloat16: the
// grouped product of the tcgen05 library between gfb_moe_gather_rows and gfb_moe_combine_rows, tiles of 128 rows) or on
// CUDA cores (32-bit, and shapes the tensor-core tiles do not take: moe_tiles_simt_kernel, tiles of 64 rows).  In every
// form a number is one sum over k in 32-bit in an order that does not depend on the other rows, so a token's result does
// not depend on what else is in the batch.
#include "common.cuh"

GFB_DEFINE_LAST_ERROR()

__device__ __forceinline__ float ldw(const void* p, int dt, size_t i) {
    return dt == GFB_BF16 ? __bfloat162float(((const __nv_bfloat16*)p)[i]) : ((const float*)p)[i];
}
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

// ------------------------------------------------------------------------------------ router ----
constexpr int MAX_EPL = 16;           // experts per lane: E <= 512
constexpr int ROUTE_WARPS = 4;
enum { ROUTE_SIGMOID = 0, ROUTE_SOFTMAX_TOP = 1 };

// one token's choice by one warp: `logits` are the token's E router logits
__device__ __forceinline__ void route_token(const float* __restrict__ logits, const void* __restrict__ correction, int c_dt, int E, int top,
                                            float scale, int* __restrict__ idx, float* __restrict__ weights, int lane, int mode) {
    float s[MAX_EPL], c[MAX_EPL];
#pragma unroll
    for (int i = 0; i < MAX_EPL; i++) {
        const int e = lane + 32 * i;
        if (e < E) {
            s[i] = mode == ROUTE_SOFTMAX_TOP ? logits[e] : sigmoid_f(logits[e]);
            c[i] = s[i] + (correction != nullptr ? ldw(correction, c_dt, e) : 0.f);
        } else {
            s[i] = 0.f;
            c[i] = -INFINITY;
        }
    }
    float sum = 0.f, mine = 0.f;       // lane r keeps the r-th chosen score
    float first = 0.f;                 // the largest chosen logit (softmax over the chosen ones)
    int mine_e = 0;
    for (int r = 0; r < top; r++) {
        float best = -INFINITY, best_s = 0.f;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < MAX_EPL; i++)
            if (c[i] > best) { best = c[i]; best_e = lane + 32 * i; best_s = s[i]; }     // ascending e per lane: the lowest index wins a tie
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o), os = __shfl_xor_sync(0xffffffffu, best_s, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; best_s = os; }
        }
#pragma unroll
        for (int i = 0; i < MAX_EPL; i++)
            if (lane + 32 * i == best_e) c[i] = -INFINITY;
        if (mode == ROUTE_SOFTMAX_TOP) {
            if (r == 0) first = best_s;
            best_s = expf(best_s - first);
        }
        sum += best_s;
        if (lane == r) { mine = best_s; mine_e = best_e; }
    }
    if (lane < top) {
        idx[lane] = mine_e;
        weights[lane] = mode == ROUTE_SOFTMAX_TOP ? mine / sum * scale : mine / (sum + 1e-20f) * scale;
    }
}

__global__ void __launch_bounds__(32 * ROUTE_WARPS)
moe_route_kernel(const float* __restrict__ logits, int ld, const void* __restrict__ correction, int c_dt, int E, int top,
                 float scale, int* __restrict__ idx, float* __restrict__ weights, int T, int mode) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * ROUTE_WARPS + (threadIdx.x >> 5);
    if (t >= T) return;
    route_token(logits + (size_t)t * ld, correction, c_dt, E, top, scale, idx + (size_t)t * top, weights + (size_t)t * top, lane, mode);
}

GFB_API int gfb_moe_route(const float* logits, int ld, const void* correction, int c_dt, int E, int top, float scale, int* idx,
                          float* weights, int T, int mode, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (E < 1 || E > 32 * MAX_EPL) return gfb_fail("gfb_moe_route: %d experts (1 to %d)", E, 32 * MAX_EPL);
    if (top < 1 || top > 32 || top > E) return gfb_fail("gfb_moe_route: %d of %d experts per token (1 to 32)", top, E);
    cudaError_t e = gfb_launch(moe_route_kernel, dim3((T + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(32 * ROUTE_WARPS), 0, stream, logits, ld,
                               correction, c_dt, E, top, scale, idx, weights, T, mode);
    return gfb_check(e, "gfb_moe_route");
}

// ------------------------------------------------------------------------------------ few tokens ----
// dot of a weight row with a staged 32-bit vector: lanes take 16 bytes of the row at a time where the row allows it
template <typename T> struct Vec;
template <> struct Vec<__nv_bfloat16> { static constexpr int N = 8; };
template <> struct Vec<float> { static constexpr int N = 4; };

template <typename T>
__device__ __forceinline__ float row_dot(const T* __restrict__ row, const float* __restrict__ v, int n, int lane, bool wide) {
    float acc = 0.f;
    if (wide) {
        constexpr int N = Vec<T>::N;
        for (int c = lane * N; c < n; c += 32 * N) {
            const uint4 raw = *reinterpret_cast<const uint4*>(row + c);
            const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
            for (int i = 0; i < N; i++) acc = fmaf(gfb_to_f32(e[i]), v[c + i], acc);
        }
    } else {
        for (int c = lane; c < n; c += 32) acc = fmaf(gfb_to_f32(row[c]), v[c], acc);
    }
    return gfb_warp_sum(acc);
}

template <typename T>
__device__ __forceinline__ bool rows_wide(const T* base, int n) {
    return n % Vec<T>::N == 0 && (reinterpret_cast<uintptr_t>(base) & 15) == 0;
}

// A decode step's router in one launch: a block per token computes the E logits (a warp per expert row, the token's input
// staged in shared memory in 32-bit) and its first warp chooses.
constexpr int ROUTER_WARPS = 8;

template <typename T>
__global__ void __launch_bounds__(32 * ROUTER_WARPS)
moe_router_kernel(const T* __restrict__ h, const T* __restrict__ router, const void* __restrict__ correction, int c_dt, int E, int top,
                  float scale, int* __restrict__ idx, float* __restrict__ weights, int D, int mode, int n_extra, float* __restrict__ extra) {
    extern __shared__ __align__(16) float rs[];        // the input [D], then the logits [E + n_extra]
    float* z = rs + D;
    gfb_pdl_launch();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x;
    gfb_pdl_wait();
    for (int i = threadIdx.x; i < D; i += blockDim.x) rs[i] = gfb_to_f32(h[(size_t)t * D + i]);
    __syncthreads();
    const bool wide = rows_wide(router, D);
    for (int e = warp; e < E + n_extra; e += ROUTER_WARPS) {
        const float d = row_dot(router + (size_t)e * D, rs, D, lane, wide);
        if (lane == 0) {
            z[e] = d;
            if (e >= E) extra[(size_t)t * n_extra + (e - E)] = d;      // rows behind the experts': their logits are handed out as they are
        }
    }
    __syncthreads();
    if (warp == 0) route_token(z, correction, c_dt, E, top, scale, idx + (size_t)t * top, weights + (size_t)t * top, lane, mode);
}

// h [T, D] and router [>= E + n_extra, D] of type dt (further rows are padding); few tokens only: a block per token.
// The logits of the n_extra rows behind the experts' go to extra float32 [T, n_extra].
GFB_API int gfb_moe_router(const void* h, const void* router, int dt, const void* correction, int c_dt, int E, int top, float scale,
                           int* idx, float* weights, int T, int D, int mode, int n_extra, float* extra, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (E < 1 || E > 32 * MAX_EPL) return gfb_fail("gfb_moe_router: %d experts (1 to %d)", E, 32 * MAX_EPL);
    if (top < 1 || top > 32 || top > E) return gfb_fail("gfb_moe_router: %d of %d experts per token (1 to 32)", top, E);
    if (n_extra < 0 || (n_extra > 0 && extra == nullptr)) return gfb_fail("gfb_moe_router: %d further rows without a place for their logits", n_extra);
    const size_t smem = (size_t)(D + E + n_extra) * sizeof(float);
    if (smem > 48 * 1024) return gfb_fail("gfb_moe_router: %zu bytes of shared memory", smem);
    cudaError_t e;
    if (dt == GFB_BF16)
        e = gfb_launch(moe_router_kernel<__nv_bfloat16>, dim3((unsigned)T), dim3(32 * ROUTER_WARPS), smem, stream, (const __nv_bfloat16*)h,
                       (const __nv_bfloat16*)router, correction, c_dt, E, top, scale, idx, weights, D, mode, n_extra, extra);
    else if (dt == GFB_F32)
        e = gfb_launch(moe_router_kernel<float>, dim3((unsigned)T), dim3(32 * ROUTER_WARPS), smem, stream, (const float*)h, (const float*)router,
                       correction, c_dt, E, top, scale, idx, weights, D, mode, n_extra, extra);
    else return gfb_fail("gfb_moe_router: unknown type %d", dt);
    return gfb_check(e, "gfb_moe_router");
}

constexpr int GEMV_WARPS = 8;
constexpr int GLU_PER_WARP = 2;       // hidden units per warp: 4 weight rows in flight

template <typename T>
__global__ void __launch_bounds__(32 * GEMV_WARPS)
moe_glu_gemv_kernel(const T* __restrict__ h, const int* __restrict__ idx, const T* __restrict__ w13, T* __restrict__ act, int top,
                    int E, int F, int D, float limit, float alpha, float shift) {
    extern __shared__ __align__(16) float hs[];
    gfb_pdl_launch();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pair = blockIdx.y, t = pair / top;
    gfb_pdl_wait();
    const int e = idx[pair];
    for (int i = threadIdx.x; i < D; i += blockDim.x) hs[i] = gfb_to_f32(h[(size_t)t * D + i]);
    __syncthreads();
    if (e < 0 || e >= E) return;
    const T* w = w13 + (size_t)e * 2 * F * D;
    const bool wide = rows_wide(w, D);
    const int f0 = (blockIdx.x * GEMV_WARPS + warp) * GLU_PER_WARP;
#pragma unroll
    for (int r = 0; r < GLU_PER_WARP; r++) {
        const int f = f0 + r;
        if (f >= F) break;
        float g = row_dot(w + (size_t)(2 * f) * D, hs, D, lane, wide);
        float u = row_dot(w + (size_t)(2 * f + 1) * D, hs, D, lane, wide);
        if (limit > 0.f) { g = fminf(g, limit); u = fminf(fmaxf(u, -limit), limit); }
        if (lane == 0) act[(size_t)pair * F + f] = gfb_from_f32<T>(g * sigmoid_f(alpha * g) * (u + shift));
    }
}

template <typename T>
__global__ void __launch_bounds__(32 * GEMV_WARPS)
moe_down_gemv_kernel(const T* __restrict__ act, const int* __restrict__ idx, const float* __restrict__ weights, const T* __restrict__ w2,
                     float* __restrict__ x, int top, int E, int F, int D) {
    extern __shared__ __align__(16) float as[];        // [top][F]
    gfb_pdl_launch();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.y;
    gfb_pdl_wait();
    for (int i = threadIdx.x; i < top * F; i += blockDim.x) as[i] = gfb_to_f32(act[(size_t)t * top * F + i]);
    __syncthreads();
    const int n = blockIdx.x * GEMV_WARPS + warp;
    if (n >= D) return;
    const bool wide = rows_wide(w2, F) && ((size_t)D * F) % Vec<T>::N == 0;
    float acc = 0.f;
    for (int r = 0; r < top; r++) {
        const int e = idx[(size_t)t * top + r];
        if (e < 0 || e >= E) continue;
        acc = fmaf(weights[(size_t)t * top + r], row_dot(w2 + ((size_t)e * D + n) * F, as + (size_t)r * F, F, lane, wide), acc);
    }
    if (lane == 0) x[(size_t)t * D + n] += acc;
}

template <typename K>
static int allow_smem(K kernel, size_t smem, const char* what) {
    if (smem > 200 * 1024) return gfb_fail("%s: %zu bytes of shared memory", what, smem);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return gfb_fail("%s: %s", what, cudaGetErrorString(e));
    }
    return 0;
}

// ------------------------------------------------------------------------------------ many tokens ----
// The plan: rows of the sorted order.  Expert e's pairs take rows start[e] .. start[e] + count[e] - 1, start[e] a
// multiple of the tile height BM; row_pair[row] is the pair of a row (-1: padding), tile_expert[tile] the expert whose
// weights a tile of that many rows uses (-1: the tile is beyond the last expert's rows), *tiles_used (if asked for) the number
// of tiles with an expert, which come first.  One block builds it; the order of an
// expert's rows among themselves is whatever the atomics give, and no result depends on it.
constexpr int PLAN_THREADS = 1024;

__global__ void __launch_bounds__(PLAN_THREADS)
moe_plan_kernel(const int* __restrict__ idx, int n_pairs, int E, int tile_rows, int* __restrict__ row_pair, int* __restrict__ pair_row,
                int* __restrict__ tile_expert, int max_tiles, int* __restrict__ tiles_used) {
    extern __shared__ int sh[];          // count[E], start[E], fill[E]
    int* count = sh;
    int* start = sh + E;
    int* fill = sh + 2 * E;
    gfb_pdl_launch();
    gfb_pdl_wait();
    for (int e = threadIdx.x; e < E; e += blockDim.x) { count[e] = 0; fill[e] = 0; }
    for (int i = threadIdx.x; i < max_tiles * tile_rows; i += blockDim.x) row_pair[i] = -1;
    for (int i = threadIdx.x; i < max_tiles; i += blockDim.x) tile_expert[i] = -1;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = idx[p];
        if (e >= 0 && e < E) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < E; e++) {
            start[e] = at;
            const int tiles = (count[e] + tile_rows - 1) / tile_rows;
            for (int i = 0; i < tiles; i++) tile_expert[at / tile_rows + i] = e;
            at += tiles * tile_rows;
        }
        if (tiles_used != nullptr) *tiles_used = at / tile_rows;       // the tiles with rows come first
    }
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = idx[p];
        if (e >= 0 && e < E) {
            const int row = start[e] + atomicAdd(&fill[e], 1);
            row_pair[row] = p;
            pair_row[p] = row;
        } else {
            pair_row[p] = -1;
        }
    }
}

GFB_API int gfb_moe_plan(const int* idx, int n_pairs, int E, int tile_rows, int* row_pair, int* pair_row, int* tile_expert, int max_tiles,
                         int* tiles_used, cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    const long busy = n_pairs < E ? n_pairs : E;             // experts that can have rows at all
    if (tile_rows < 1 || (long)max_tiles < ((long)n_pairs + busy * (tile_rows - 1)) / tile_rows)
        return gfb_fail("gfb_moe_plan: %d tiles of %d rows cannot hold %d pairs of %d experts", max_tiles, tile_rows, n_pairs, E);
    const size_t smem = (size_t)3 * E * sizeof(int);
    cudaError_t e = gfb_launch(moe_plan_kernel, dim3(1), dim3(PLAN_THREADS), smem, stream, idx, n_pairs, E, tile_rows, row_pair, pair_row,
                               tile_expert, max_tiles, tiles_used);
    return gfb_check(e, "gfb_moe_plan");
}

// Tiles on CUDA cores (the 32-bit path, and bfloat16 shapes the tensor-core tiles do not take): 64 x 64 outputs per block,
// each one thread's ascending sum over k.  GLU: A = h rows gathered by pair / top, W = w13 of the tile's expert, the
// output act[row, n / 2] from the gate (even n) and up (odd n) columns.  DOWN: A = act rows (sorted order), W = w2 of
// the tile's expert, the output y[pair, n] in 32-bit, pair order.
constexpr int BM = 64, BN = 64, BK = 16;

template <typename T, bool GLU>
__global__ void __launch_bounds__(256)
moe_tiles_simt_kernel(const T* __restrict__ A, const T* __restrict__ W, void* __restrict__ C, const int* __restrict__ row_pair,
                      const int* __restrict__ tile_expert, int top, int N, int K, float limit, float alpha, float shift) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    __shared__ int src_row[BM];
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int e = tile_expert[blockIdx.y];
    if (e < 0) return;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    if (threadIdx.x < BM) {
        const int p = row_pair[m0 + threadIdx.x];
        src_row[threadIdx.x] = p < 0 ? -1 : (GLU ? p / top : m0 + (int)threadIdx.x);
    }
    __syncthreads();
    const T* We = W + (size_t)e * N * K;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int el = threadIdx.x + i * 256;
            const int r = el >> 4, k = el & 15;
            const int gk = k0 + k, gn = n0 + r, sr = src_row[r];
            As[k][r] = (sr >= 0 && gk < K) ? gfb_to_f32(A[(size_t)sr * K + gk]) : 0.f;
            Ws[k][r] = (gn < N && gk < K) ? gfb_to_f32(We[(size_t)gn * K + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; k++) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) w[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int r = ty * 4 + i;
        const int p = row_pair[m0 + r];
        if (p < 0) continue;
        if (GLU) {
            T* out = (T*)C + (size_t)(m0 + r) * (N >> 1);
#pragma unroll
            for (int j = 0; j < 4; j += 2) {
                const int n = n0 + tx * 4 + j;
                if (n + 1 < N) {
                    float g = acc[i][j], u = acc[i][j + 1];
                    if (limit > 0.f) { g = fminf(g, limit); u = fminf(fmaxf(u, -limit), limit); }
                    out[n >> 1] = gfb_from_f32<T>(g * sigmoid_f(alpha * g) * (u + shift));
                }
            }
        } else {
            float* out = (float*)C + (size_t)p * N;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int n = n0 + tx * 4 + j;
                if (n < N) out[n] = acc[i][j];
            }
        }
    }
}

// x[t] += sum_r weights[t, r] * y[t * top + r] in ascending r
__global__ void moe_combine_kernel(const float* __restrict__ y, const float* __restrict__ weights, float* __restrict__ x, int top,
                                   int D, long n) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long t = i / D;
    const int c = (int)(i - t * D);
    float acc = 0.f;
    for (int r = 0; r < top; r++) acc = fmaf(weights[t * top + r], y[((size_t)t * top + r) * D + c], acc);
    x[i] += acc;
}

// ------------------------------------------------------------------------------------ around the tensor-core tiles ----
// The tensor cores' tiles read their rows where TMA finds them: side by side in the sorted order.  hs[row] = h[row_pair[row] / top]
// (zeros for padding rows), 16 bytes per thread and step.
__global__ void __launch_bounds__(128)
moe_gather_rows_kernel(const uint4* __restrict__ h, const int* __restrict__ row_pair, uint4* __restrict__ hs, int top, int vec_per_row) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int row = blockIdx.x;
    const int p = row_pair[row];
    const uint4* src = p < 0 ? nullptr : h + (size_t)(p / top) * vec_per_row;
    uint4* dst = hs + (size_t)row * vec_per_row;
    for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) dst[i] = src ? src[i] : make_uint4(0u, 0u, 0u, 0u);
}

// h [T, D] bfloat16 with D % 8 == 0 -> hs [rows, D] in the plan's sorted order
GFB_API int gfb_moe_gather_rows(const void* h, const int* row_pair, void* hs, int rows, int top, int D, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (D % 8 || ((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(hs)) & 15))
        return gfb_fail("gfb_moe_gather_rows: rows of %d bfloat16 numbers are not whole 16-byte pieces", D);
    cudaError_t e = gfb_launch(moe_gather_rows_kernel, dim3((unsigned)rows), dim3(128), 0, stream, (const uint4*)h, row_pair, (uint4*)hs, top,
                               D / 8);
    return gfb_check(e, "gfb_moe_gather_rows");
}

// x[t] += sum_r weights[t, r] * y[pair_row[t * top + r]] in ascending r; y in the plan's sorted order, D % 4 == 0
__global__ void __launch_bounds__(256)
moe_combine_rows_kernel(const float4* __restrict__ y, const int* __restrict__ pair_row, const float* __restrict__ weights,
                        float4* __restrict__ x, int top, int vec_per_row, long n) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long t = i / vec_per_row;
    const int c = (int)(i - t * vec_per_row);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < top; r++) {
        const int row = pair_row[t * top + r];
        if (row < 0) continue;
        const float w = weights[t * top + r];
        const float4 v = y[(size_t)row * vec_per_row + c];
        acc.x = fmaf(w, v.x, acc.x); acc.y = fmaf(w, v.y, acc.y); acc.z = fmaf(w, v.z, acc.z); acc.w = fmaf(w, v.w, acc.w);
    }
    float4 o = x[i];
    o.x += acc.x; o.y += acc.y; o.z += acc.z; o.w += acc.w;
    x[i] = o;
}

GFB_API int gfb_moe_combine_rows(const float* y, const int* pair_row, const float* weights, float* x, int T, int top, int D,
                                 cudaStream_t stream) {
    if (T <= 0) return 0;
    if (D % 4 || ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(x)) & 15))
        return gfb_fail("gfb_moe_combine_rows: rows of %d floats are not whole 16-byte pieces", D);
    const long n = (long)T * (D / 4);
    cudaError_t e = gfb_launch(moe_combine_rows_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, (const float4*)y, pair_row,
                               weights, (float4*)x, top, D / 4, n);
    return gfb_check(e, "gfb_moe_combine_rows");
}

// h [T, D], w13 [E, 2F, D], act [rows, F] of type dt.  tiles = 0: the few-token form, act in pair order (rows = T * top);
// otherwise act in the plan's sorted order (rows = max_tiles * 64) and row_pair, tile_expert from gfb_moe_plan with tiles of 64 rows.
GFB_API int gfb_moe_glu(const void* h, const int* idx, const void* w13, void* act, int dt, int T, int top, int E, int F, int D,
                        float limit, float alpha, float shift, const int* row_pair, const int* tile_expert, int max_tiles,
                        cudaStream_t stream) {
    if (T <= 0) return 0;
    typedef __nv_bfloat16 bf16;
    cudaError_t e;
    if (max_tiles > 0) {
        dim3 grid((2 * F + BN - 1) / BN, max_tiles);
        if (max_tiles > 65535) return gfb_fail("gfb_moe_glu: %d tiles exceed the grid limit", max_tiles);
        if (dt == GFB_BF16)
            e = gfb_launch(moe_tiles_simt_kernel<bf16, true>, grid, dim3(256), 0, stream, (const bf16*)h, (const bf16*)w13, act, row_pair,
                           tile_expert, top, 2 * F, D, limit, alpha, shift);
        else if (dt == GFB_F32)
            e = gfb_launch(moe_tiles_simt_kernel<float, true>, grid, dim3(256), 0, stream, (const float*)h, (const float*)w13, act, row_pair,
                           tile_expert, top, 2 * F, D, limit, alpha, shift);
        else return gfb_fail("gfb_moe_glu: unknown type %d", dt);
        return gfb_check(e, "gfb_moe_glu (tiles)");
    }
    const long pairs = (long)T * top;
    if (pairs > 65535) return gfb_fail("gfb_moe_glu: %ld pairs exceed the grid limit of the few-token form", pairs);
    const size_t smem = (size_t)D * sizeof(float);
    dim3 grid((F + GEMV_WARPS * GLU_PER_WARP - 1) / (GEMV_WARPS * GLU_PER_WARP), (unsigned)pairs);
    if (dt == GFB_BF16) {
        if (allow_smem(moe_glu_gemv_kernel<bf16>, smem, "gfb_moe_glu")) return 1;
        e = gfb_launch(moe_glu_gemv_kernel<bf16>, grid, dim3(32 * GEMV_WARPS), smem, stream, (const bf16*)h, idx, (const bf16*)w13, (bf16*)act,
                       top, E, F, D, limit, alpha, shift);
    } else if (dt == GFB_F32) {
        if (allow_smem(moe_glu_gemv_kernel<float>, smem, "gfb_moe_glu")) return 1;
        e = gfb_launch(moe_glu_gemv_kernel<float>, grid, dim3(32 * GEMV_WARPS), smem, stream, (const float*)h, idx, (const float*)w13,
                       (float*)act, top, E, F, D, limit, alpha, shift);
    } else return gfb_fail("gfb_moe_glu: unknown type %d", dt);
    return gfb_check(e, "gfb_moe_glu");
}

// act as gfb_moe_glu left it; w2 [E, D, F]; x float32 [T, D] += the weighted sum of the chosen experts' outputs.
// With tiles: y float32 [T * top, D] is scratch for the experts' outputs in pair order.
GFB_API int gfb_moe_down(const void* act, const int* idx, const float* weights, const void* w2, float* x, int dt, int T, int top,
                         int E, int F, int D, const int* row_pair, const int* tile_expert, int max_tiles, float* y,
                         cudaStream_t stream) {
    if (T <= 0) return 0;
    typedef __nv_bfloat16 bf16;
    cudaError_t e;
    if (max_tiles > 0) {
        dim3 grid((D + BN - 1) / BN, max_tiles);
        if (dt == GFB_BF16)
            e = gfb_launch(moe_tiles_simt_kernel<bf16, false>, grid, dim3(256), 0, stream, (const bf16*)act, (const bf16*)w2, (void*)y,
                           row_pair, tile_expert, top, D, F, 0.f, 0.f, 0.f);
        else if (dt == GFB_F32)
            e = gfb_launch(moe_tiles_simt_kernel<float, false>, grid, dim3(256), 0, stream, (const float*)act, (const float*)w2, (void*)y,
                           row_pair, tile_expert, top, D, F, 0.f, 0.f, 0.f);
        else return gfb_fail("gfb_moe_down: unknown type %d", dt);
        if (gfb_check(e, "gfb_moe_down (tiles)")) return 1;
        const long n = (long)T * D;
        e = gfb_launch(moe_combine_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, (const float*)y, weights, x, top, D, n);
        return gfb_check(e, "gfb_moe_down (combine)");
    }
    if (T > 65535) return gfb_fail("gfb_moe_down: %d tokens exceed the grid limit of the few-token form", T);
    const size_t smem = (size_t)top * F * sizeof(float);
    dim3 grid((D + GEMV_WARPS - 1) / GEMV_WARPS, T);
    if (dt == GFB_BF16) {
        if (allow_smem(moe_down_gemv_kernel<bf16>, smem, "gfb_moe_down")) return 1;
        e = gfb_launch(moe_down_gemv_kernel<bf16>, grid, dim3(32 * GEMV_WARPS), smem, stream, (const bf16*)act, idx, weights, (const bf16*)w2,
                       x, top, E, F, D);
    } else if (dt == GFB_F32) {
        if (allow_smem(moe_down_gemv_kernel<float>, smem, "gfb_moe_down")) return 1;
        e = gfb_launch(moe_down_gemv_kernel<float>, grid, dim3(32 * GEMV_WARPS), smem, stream, (const float*)act, idx, weights,
                       (const float*)w2, x, top, E, F, D);
    } else return gfb_fail("gfb_moe_down: unknown type %d", dt);
    return gfb_check(e, "gfb_moe_down");
}
