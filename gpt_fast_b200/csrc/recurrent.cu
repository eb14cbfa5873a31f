// Kernels of recurrent mixers whose state is a matrix per head, carried from token to token in 32-bit:
//
// gfb_short_conv    causal convolution over time per channel (a few taps, optional bias) and SiLU; the last
//                   taps - 1 inputs of every sequence are state, so a sequence may arrive in any portions
// gfb_ssd_scan      selective state space with a scalar decay per head and token:
//                       dt = softplus(dt_raw + dt_bias_h),  S <- exp(-exp(A_log_h) dt) S + dt B x^T,  y = S^T C + D_h x
// gfb_delta_rule    gated delta rule with a decay per head and key channel:
//                       S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//                   with q, k made unit vectors per head (q also times dim^-1/2), beta = sigmoid(.),
//                   g = exp(-exp(A_log_h) softplus(a_raw + dt_bias))
// gfb_gated_norm    root-mean-square norm over groups of columns with a weight and a gate (SiLU or sigmoid) that
//                   is applied before or behind the norm
// gfb_rglru         a gated linear recurrence per channel (the real-gated linear recurrent unit): with the channels in
//                   equal blocks and a square matrix per block and gate,
//                       r = sigmoid(Wa_b u_b + ba),  i = sigmoid(Wi_b u_b + bi),  a = exp(-c r softplus(lam)),
//                       S <- a S + sqrt(1 - a^2) i u,   out = S * gelu_tanh(y + by)
//                   S one number per channel and sequence, 32-bit
//
// The two recurrences share one layout: a block owns one (sequence, head) and a slice of the state's columns and
// walks through the sequence's tokens of this step; a lane keeps RPT rows of one column of S in registers.  Sums
// over the rows are added per lane in ascending order and then over the lanes of the column in a fixed butterfly, so
// a token's result is the same bits however the sequence was cut into steps or batched.  Everything is 32-bit.
#include "common.cuh"

GFB_DEFINE_LAST_ERROR()

__device__ __forceinline__ float ldw(const void* p, int dt, size_t i) {
    return dt == GFB_BF16 ? __bfloat162float(((const __nv_bfloat16*)p)[i]) : ((const float*)p)[i];
}
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }

// ------------------------------------------------------------------------------ short convolution ----
constexpr int MAX_TAPS = 16;

// state of a slot: [taps - 1][C] inputs, oldest first, at state + slot * state_ld
template <typename T>
__global__ void short_conv_kernel(const T* __restrict__ src, int ld, int col_off, int C, const void* __restrict__ w,
                                  const void* __restrict__ bias, const void* __restrict__ in_bias, int w_dt, int taps,
                                  const float* __restrict__ state, size_t state_ld, float* __restrict__ out, GfbBatch b, int act) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int s = b.tok_seq[t];
    const int i = t - b.cu_seqlens[s];
    const float* st = state + (size_t)b.slots[s] * state_ld;
    float acc = bias != nullptr ? ldw(bias, w_dt, c) : 0.f;
    const float ib = in_bias != nullptr ? ldw(in_bias, w_dt, c) : 0.f;       // part of every real input, not of the zeros ahead of a sequence
    for (int j = 0; j < taps; j++) {
        const int back = taps - 1 - j;
        float v;
        if (i - back >= 0) v = gfb_to_f32(src[(size_t)(t - back) * ld + col_off + c]) + ib;
        else v = st[(size_t)(taps - 1 + i - back) * C + c];
        acc = fmaf(ldw(w, w_dt, (size_t)c * taps + j), v, acc);
    }
    out[(size_t)t * C + c] = act ? silu_f(acc) : acc;
}

template <typename T>
__global__ void conv_state_kernel(const T* __restrict__ src, int ld, int col_off, int C, const void* __restrict__ in_bias, int w_dt,
                                  int taps, float* __restrict__ state, size_t state_ld, GfbBatch b) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int s = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int t0 = b.cu_seqlens[s], n = b.cu_seqlens[s + 1] - t0;
    float* st = state + (size_t)b.slots[s] * state_ld;
    float keep[MAX_TAPS];
    const float ib = in_bias != nullptr ? ldw(in_bias, w_dt, c) : 0.f;
#pragma unroll
    for (int k = 0; k < MAX_TAPS; k++) {
        if (k < taps - 1) {
            const int i = n - (taps - 1) + k;                   // index among this step's tokens; negative: older
            keep[k] = i >= 0 ? gfb_to_f32(src[(size_t)(t0 + i) * ld + col_off + c]) + ib : st[(size_t)(taps - 1 + i) * C + c];
        }
    }
#pragma unroll
    for (int k = 0; k < MAX_TAPS; k++)
        if (k < taps - 1) st[(size_t)k * C + c] = keep[k];
}

// src [T, ld] of type dt, C channels from column col_off; w [C, taps] and bias [C] (or null) of type w_dt;
// state float32, slot stride state_ld, (taps - 1) * C numbers per slot; out float32 [T, C]; act: 1 = SiLU, 0 = none.
// in_bias [C] (or null) is added to every input before the taps (the state keeps the sums).
// The state is advanced by a second kernel behind the first.
GFB_API int gfb_short_conv(const void* src, int dt, int ld, int col_off, int C, const void* w, const void* bias, const void* in_bias, int w_dt,
                           int taps, float* state, long state_ld, float* out, const int* cu_seqlens, const int* tok_seq,
                           const int* slots, const int* lengths, int n_seqs, int n_tokens, int act, cudaStream_t stream) {
    if (n_tokens <= 0 || C <= 0) return 0;
    if (taps < 1 || taps > MAX_TAPS) return gfb_fail("gfb_short_conv: %d taps (1 to %d)", taps, MAX_TAPS);
    GfbBatch b{cu_seqlens, tok_seq, slots, lengths, n_seqs, n_tokens};
    const int threads = 128;
    const unsigned cb = (unsigned)((C + threads - 1) / threads);
    if (cb > 65535) return gfb_fail("gfb_short_conv: %d channels exceed the grid limit", C);
    cudaError_t e;
    if (dt == GFB_BF16)
        e = gfb_launch(short_conv_kernel<__nv_bfloat16>, dim3(n_tokens, cb), dim3(threads), 0, stream, (const __nv_bfloat16*)src, ld,
                       col_off, C, w, bias, in_bias, w_dt, taps, (const float*)state, (size_t)state_ld, out, b, act);
    else if (dt == GFB_F32)
        e = gfb_launch(short_conv_kernel<float>, dim3(n_tokens, cb), dim3(threads), 0, stream, (const float*)src, ld, col_off, C, w,
                       bias, in_bias, w_dt, taps, (const float*)state, (size_t)state_ld, out, b, act);
    else
        return gfb_fail("gfb_short_conv: unknown type %d", dt);
    if (gfb_check(e, "gfb_short_conv")) return 1;
    if (taps == 1) return 0;
    if (dt == GFB_BF16)
        e = gfb_launch(conv_state_kernel<__nv_bfloat16>, dim3(n_seqs, cb), dim3(threads), 0, stream, (const __nv_bfloat16*)src, ld,
                       col_off, C, in_bias, w_dt, taps, state, (size_t)state_ld, b);
    else
        e = gfb_launch(conv_state_kernel<float>, dim3(n_seqs, cb), dim3(threads), 0, stream, (const float*)src, ld, col_off, C, in_bias, w_dt, taps,
                       state, (size_t)state_ld, b);
    return gfb_check(e, "gfb_short_conv (state)");
}

// ------------------------------------------------------------------------------ the two recurrences ----
// Layout of both: the state of a head is rows x columns (rows: state or key channels; columns: value channels); its
// columns evolve independently, so a block takes one (sequence, head) and a slice of the columns and walks through
// the sequence's tokens of this step.  The rows are dealt in groups of RPT to RG lanes of a warp (RG a power of two),
// a warp holds 32 / RG columns, a block four warps.  A sum over the rows is RPT terms per lane in ascending order and
// then either a butterfly over the RG lanes (the delta rule's S^T k, which the token's own update waits for) or, for the
// outputs, which nothing waits for, the lanes' parts left in shared memory and added in ascending order behind the
// tile's steps: no barrier per token.  The inputs of TB tokens are staged in shared memory at a
// time (row vectors padded per group so that the RG lanes read distinct banks with 16-byte loads), in two stages: the next
// tile's copies (cp.async) run under the current tile's steps.
constexpr int TB = 16;
constexpr int SCAN_WARPS = 4;

__device__ __forceinline__ float group_sum(float v, int RG) {
    for (int o = RG >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
constexpr int ROW_PAD = 4;            // numbers of padding per group of RPT rows: 16-byte loads of a group stay aligned and
                                      // the lanes of a column fall into distinct banks
// the lanes' parts of a column's sum, in ascending order
__device__ __forceinline__ float sum_parts(const float* part, int RG) {
    float v = part[0];
    for (int r = 1; r < RG; r++) v += part[r];
    return v;
}
__device__ __forceinline__ int padded(int c, int RPT) { return c + (c / RPT) * ROW_PAD; }      // index of row c in a padded row vector
// RPT consecutive numbers of shared memory into registers, four at a time
template <int RPT>
__device__ __forceinline__ void load_rows(float (&r)[RPT], const float* p) {
#pragma unroll
    for (int i = 0; i < RPT; i += 4) {
        const float4 v = *reinterpret_cast<const float4*>(p + i);
        r[i] = v.x; r[i + 1] = v.y; r[i + 2] = v.z; r[i + 3] = v.w;
    }
}
// One 32-bit number from global to shared memory without passing a register: a tile's copies are all in flight at once
// and the next tile's run under the current tile's steps.
__device__ __forceinline__ void copy_async4(float* smem, const float* gmem) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(a), "l"(gmem));
}
__device__ __forceinline__ void copy_async16(float* smem, const float* gmem) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(a), "l"(gmem));
}
__device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
__device__ __forceinline__ void copy_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void copy_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// x [T, ldx] float32: head h's P inputs at column h * P, group g's N numbers of B at b_off + g * N, of C at
// c_off + g * N.  dt_raw: [T, ld_dt] of type TD, head h at column dt_off + h.
template <typename TD, int RPT>
__global__ void __launch_bounds__(32 * SCAN_WARPS)
ssd_scan_kernel(const float* __restrict__ x, int ldx, int b_off, int c_off, const TD* __restrict__ dt_raw, int ld_dt,
                int dt_off, const void* __restrict__ dt_bias, const void* __restrict__ a_log, const void* __restrict__ skip,
                int w_dt, float* __restrict__ state, size_t state_ld, float* __restrict__ out, GfbBatch b, int H, int P, int N,
                int G, int RG) {
    extern __shared__ __align__(16) float sm[];
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y, g = h / (H / G);
    const int CW = 32 / RG, CB = SCAN_WARPS * CW, NP = RG * (RPT + ROW_PAD);
    const int STAGE = TB * (2 * NP + CB + 2);
    float* sO = sm + 2 * STAGE;           // [TB][CB]; ahead of it two stages of: B [TB][NP], C [TB][NP], x [TB][CB], dt [TB], decay [TB]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rgi = lane % RG, cl = warp * CW + lane / RG;           // row group, column within the block
    const int p0 = blockIdx.z * CB, p = p0 + cl;
    const bool active = p < P;
    const int t0 = b.cu_seqlens[s], t1 = b.cu_seqlens[s + 1];
    float* S = state + (size_t)b.slots[s] * state_ld + (size_t)h * N * P;
    float st[RPT];
#pragma unroll
    for (int r = 0; r < RPT; r++) {
        const int n = rgi * RPT + r;
        st[r] = (active && n < N) ? S[(size_t)n * P + p] : 0.f;
    }
    const float bias = ldw(dt_bias, w_dt, h), rate = expf(ldw(a_log, w_dt, h)), dskip = skip != nullptr ? ldw(skip, w_dt, h) : 0.f;
    // rows and columns beyond the state's stay zero: clear the token rows this step will use, in the stages it will use
    {
        const int used = min(TB, t1 - t0), stages = t1 - t0 > TB ? 2 : 1;
        for (int st_ = 0; st_ < stages; st_++) {
            float* base = sm + st_ * STAGE;
            for (int i = tid; i < used * NP; i += blockDim.x) { base[i] = 0.f; base[TB * NP + i] = 0.f; }
            for (int i = tid; i < used * CB; i += blockDim.x) base[2 * TB * NP + i] = 0.f;
        }
    }
    __syncthreads();
    float dt_next = 0.f;
    const bool wide = N % 4 == 0 && ldx % 4 == 0 && aligned16(x + b_off + g * N) && aligned16(x + c_off + g * N);
    auto fetch = [&](int stage, int tile) {
        float* base = sm + stage * STAGE;
        const int nt = min(TB, t1 - tile);
        for (int tt = warp; tt < nt; tt += SCAN_WARPS) {
            const float* row = x + (size_t)(tile + tt) * ldx;
            if (wide) {                                            // four numbers per copy (a group of RPT rows is contiguous)
                for (int n = 4 * lane; n < N; n += 128) {
                    copy_async16(base + tt * NP + padded(n, RPT), row + b_off + g * N + n);
                    copy_async16(base + TB * NP + tt * NP + padded(n, RPT), row + c_off + g * N + n);
                }
            } else {
                for (int n = lane; n < N; n += 32) {
                    copy_async4(base + tt * NP + padded(n, RPT), row + b_off + g * N + n);
                    copy_async4(base + TB * NP + tt * NP + padded(n, RPT), row + c_off + g * N + n);
                }
            }
            for (int q = lane; q < CB && p0 + q < P; q += 32) copy_async4(base + 2 * TB * NP + tt * CB + q, row + (size_t)h * P + p0 + q);
        }
        copy_commit();
        if (tid < nt) dt_next = gfb_to_f32(dt_raw[(size_t)(tile + tid) * ld_dt + dt_off + h]);
    };
    if (t0 < t1) fetch(0, t0);
    int stage = 0;
    for (int tile = t0; tile < t1; tile += TB, stage ^= 1) {
        const int nt = min(TB, t1 - tile);
        float* sB = sm + stage * STAGE;
        float* sC = sB + TB * NP;
        float* sX = sC + TB * NP;
        float* sDt = sX + TB * CB;
        float* sA = sDt + TB;
        if (tid < nt) {
            const float d = softplus_f(dt_next + bias);
            sDt[tid] = d;
            sA[tid] = expf(-rate * d);
        }
        if (tile + TB < t1) {
            fetch(stage ^ 1, tile + TB);                       // runs under this tile's steps
            copy_wait<1>();
        } else {
            copy_wait<0>();
        }
        __syncthreads();                                       // this tile's inputs have landed; the previous outputs are written
        for (int tt = 0; tt < nt; tt++) {
            const float a = sA[tt], dx = sDt[tt], xp = sX[tt * CB + cl];
            float bb[RPT], cc[RPT];
            load_rows<RPT>(bb, sB + tt * NP + rgi * (RPT + ROW_PAD));
            load_rows<RPT>(cc, sC + tt * NP + rgi * (RPT + ROW_PAD));
            float acc = 0.f;
#pragma unroll
            for (int r = 0; r < RPT; r++) {
                st[r] = fmaf(a, st[r], (dx * bb[r]) * xp);
                acc = fmaf(st[r], cc[r], acc);
            }
            acc = group_sum(acc, RG);                // (leaving the lanes' parts in shared memory as the delta rule does costs a
            if (rgi == 0) sO[tt * CB + cl] = acc + dskip * xp;      //  fourth block per SM its room, and with it a second round of blocks)
        }
        __syncthreads();
        for (int tt = warp; tt < nt; tt += SCAN_WARPS)
            for (int q = lane; q < CB; q += 32)
                if (p0 + q < P) out[(size_t)(tile + tt) * H * P + (size_t)h * P + p0 + q] = sO[tt * CB + q];
        // the next pass's barrier comes before any lane writes sO or this stage again
    }
    if (active) {
#pragma unroll
        for (int r = 0; r < RPT; r++) {
            const int n = rgi * RPT + r;
            if (n < N) S[(size_t)n * P + p] = st[r];
        }
    }
}

// What does not depend on the state is done for all tokens at once, in place: q and k become unit vectors per head
// (q also times q_scale), the decay inputs become the decays g = exp(-exp(A_log_h) softplus(a + dt_bias)).
__global__ void delta_prepare_kernel(float* __restrict__ qkv, int ldq, int q_off, int k_off, float* __restrict__ a_raw, int ld_a,
                                     int a_off, const void* __restrict__ dt_bias, const void* __restrict__ a_log, int w_dt, int H,
                                     int KH, int d, float q_scale, float unit_eps, int head_decay) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    for (int item = warp; item < 2 * KH; item += nwarp) {
        float* vec = qkv + (size_t)t * ldq + (item & 1 ? k_off : q_off) + (size_t)(item >> 1) * d;
        float ss = 0.f;
        for (int c = lane; c < d; c += 32) ss = fmaf(vec[c], vec[c], ss);
        ss = gfb_warp_sum(ss);
        const float f = (1.0f / sqrtf(ss + unit_eps)) * (item & 1 ? 1.0f : q_scale);
        for (int c = lane; c < d; c += 32) vec[c] *= f;
    }
    float* ar = a_raw + (size_t)t * ld_a + a_off;
    if (head_decay) {                                          // one decay per head: H numbers per token
        for (int h = threadIdx.x; h < H; h += blockDim.x)
            ar[h] = expf(-expf(ldw(a_log, w_dt, h)) * softplus_f(ar[h] + ldw(dt_bias, w_dt, h)));
        return;
    }
    for (int h = 0; h < H; h++) {
        const float rate = expf(ldw(a_log, w_dt, h));
        for (int c = threadIdx.x; c < d; c += blockDim.x)
            ar[(size_t)h * d + c] = expf(-rate * softplus_f(ar[(size_t)h * d + c] + ldw(dt_bias, w_dt, (size_t)h * d + c)));
    }
}

// qkv [T, ldq] float32 (convolved, activated, q and k unit vectors): query head j at q_off + j * d, key head j at
// k_off + j * d, value head h at v_off + h * dv.  beta_raw [T, ld_b] of type TD, head h at column beta_off + h.
// decay [T, ld_a] float32, head h's d channels at a_off + h * d; with head_decay one number per head, at a_off + h.
template <typename TD, int RPT>
__global__ void __launch_bounds__(32 * SCAN_WARPS)
delta_rule_kernel(const float* __restrict__ qkv, int ldq, int q_off, int k_off, int v_off, const TD* __restrict__ beta_raw, int ld_b,
                  int beta_off, const float* __restrict__ decay, int ld_a, int a_off, float* __restrict__ state, size_t state_ld,
                  float* __restrict__ out, GfbBatch b, int H, int KH, int d, int dv, int RG, int head_decay) {
    extern __shared__ __align__(16) float sm[];
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y, kh = h / (H / KH);
    const int CW = 32 / RG, CB = SCAN_WARPS * CW, NP = RG * (RPT + ROW_PAD);
    const int STAGE = TB * (3 * NP + CB + 1);
    float* sO = sm + 2 * STAGE;           // [TB][CB][RG] the lanes' parts of the outputs; ahead of it two stages of: q, k, decay [TB][NP] each, v [TB][CB], beta [TB]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rgi = lane % RG, cl = warp * CW + lane / RG;
    const int p0 = blockIdx.z * CB, p = p0 + cl;
    const bool active = p < dv;
    const int t0 = b.cu_seqlens[s], t1 = b.cu_seqlens[s + 1];
    float* S = state + (size_t)b.slots[s] * state_ld + (size_t)h * d * dv;
    float st[RPT];
#pragma unroll
    for (int r = 0; r < RPT; r++) {
        const int i = rgi * RPT + r;
        st[r] = (active && i < d) ? S[(size_t)i * dv + p] : 0.f;
    }
    // rows and columns beyond the state's stay zero: clear the token rows this step will use, in the stages it will use
    {
        const int used = min(TB, t1 - t0), stages = t1 - t0 > TB ? 2 : 1;
        for (int st_ = 0; st_ < stages; st_++) {
            float* base = sm + st_ * STAGE;
            for (int i = tid; i < used * NP; i += blockDim.x) { base[i] = 0.f; base[TB * NP + i] = 0.f; base[2 * TB * NP + i] = 0.f; }
            for (int i = tid; i < used * CB; i += blockDim.x) base[3 * TB * NP + i] = 0.f;
        }
    }
    __syncthreads();
    float beta_next = 0.f;
    const bool wide = d % 4 == 0 && ldq % 4 == 0 && aligned16(qkv + q_off + kh * d) && aligned16(qkv + k_off + kh * d) &&
                      (head_decay || (ld_a % 4 == 0 && aligned16(decay + a_off + (size_t)h * d)));
    auto fetch = [&](int stage, int tile) {
        float* base = sm + stage * STAGE;
        const int nt = min(TB, t1 - tile);
        for (int tt = warp; tt < nt; tt += SCAN_WARPS) {
            const float* row = qkv + (size_t)(tile + tt) * ldq;
            const float* grow = decay + (size_t)(tile + tt) * ld_a + a_off + (head_decay ? (size_t)h : (size_t)h * d);
            if (head_decay) {                                      // the head's one decay stands in every row's place
                const float g = grow[0];
                for (int c = lane; c < d; c += 32) base[2 * TB * NP + tt * NP + padded(c, RPT)] = g;
            }
            if (wide) {                                            // four numbers per copy (a group of RPT rows is contiguous)
                for (int c = 4 * lane; c < d; c += 128) {
                    const int at = tt * NP + padded(c, RPT);
                    copy_async16(base + at, row + q_off + kh * d + c);
                    copy_async16(base + TB * NP + at, row + k_off + kh * d + c);
                    if (!head_decay) copy_async16(base + 2 * TB * NP + at, grow + c);
                }
            } else {
                for (int c = lane; c < d; c += 32) {
                    const int at = tt * NP + padded(c, RPT);
                    copy_async4(base + at, row + q_off + kh * d + c);
                    copy_async4(base + TB * NP + at, row + k_off + kh * d + c);
                    if (!head_decay) copy_async4(base + 2 * TB * NP + at, grow + c);
                }
            }
            for (int c = lane; c < CB && p0 + c < dv; c += 32) copy_async4(base + 3 * TB * NP + tt * CB + c, row + v_off + (size_t)h * dv + p0 + c);
        }
        copy_commit();
        if (tid < nt) beta_next = gfb_to_f32(beta_raw[(size_t)(tile + tid) * ld_b + beta_off + h]);
    };
    if (t0 < t1) fetch(0, t0);
    int stage = 0;
    for (int tile = t0; tile < t1; tile += TB, stage ^= 1) {
        const int nt = min(TB, t1 - tile);
        float* sQ = sm + stage * STAGE;
        float* sK = sQ + TB * NP;
        float* sG = sK + TB * NP;
        float* sV = sG + TB * NP;
        float* sBeta = sV + TB * CB;
        if (tid < nt) sBeta[tid] = sigmoid_f(beta_next);
        if (tile + TB < t1) {
            fetch(stage ^ 1, tile + TB);                       // runs under this tile's steps
            copy_wait<1>();
        } else {
            copy_wait<0>();
        }
        __syncthreads();                                       // this tile's inputs have landed; the previous outputs are written
        for (int tt = 0; tt < nt; tt++) {
            float gg[RPT], kr[RPT], qq[RPT];
            load_rows<RPT>(gg, sG + tt * NP + rgi * (RPT + ROW_PAD));
            load_rows<RPT>(kr, sK + tt * NP + rgi * (RPT + ROW_PAD));
            load_rows<RPT>(qq, sQ + tt * NP + rgi * (RPT + ROW_PAD));
            float acc = 0.f;
#pragma unroll
            for (int r = 0; r < RPT; r++) {
                st[r] *= gg[r];
                acc = fmaf(st[r], kr[r], acc);
            }
            acc = group_sum(acc, RG);
            const float u = sBeta[tt] * (sV[tt * CB + cl] - acc);
            float o = 0.f;
#pragma unroll
            for (int r = 0; r < RPT; r++) {
                st[r] = fmaf(kr[r], u, st[r]);
                o = fmaf(st[r], qq[r], o);
            }
            // nothing of the next token waits for this sum: the lanes leave their parts, added behind the tile's steps
            sO[(tt * CB + cl) * RG + rgi] = o;
        }
        __syncthreads();
        for (int tt = warp; tt < nt; tt += SCAN_WARPS)
            for (int c = lane; c < CB; c += 32)
                if (p0 + c < dv) out[(size_t)(tile + tt) * H * dv + (size_t)h * dv + p0 + c] = sum_parts(sO + (tt * CB + c) * RG, RG);
    }
    if (active) {
#pragma unroll
        for (int r = 0; r < RPT; r++) {
            const int i = rgi * RPT + r;
            if (i < d) S[(size_t)i * dv + p] = st[r];
        }
    }
}

// rows per lane and lanes per column for a state of `rows` rows: the fewest rows per lane that need at most 32 lanes
// (a token's step is a chain of dependent instructions, so few rows per lane and many lanes per column make it short;
// 128 rows: 8 rows on each of 16 lanes took 0.27 us per token where 16 rows on 8 lanes took 1.0); 0 if none does
static int pick_rpt(int rows, int* rg, bool many_blocks) {
    // with hundreds of (sequence, head) pairs the SMs are busy anyway: 16 rows per lane then halve the number of blocks
    const int rpt[4] = {8, 16, 32, 64};
    for (int i = many_blocks ? 1 : 0; i < 4; i++) {
        const int need = (rows + rpt[i] - 1) / rpt[i];
        if (need <= 32) {
            int g = 1;
            while (g < need) g <<= 1;
            *rg = g;
            return rpt[i];
        }
    }
    return 0;
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

// state float32: slot stride state_ld, per slot [H][N][P]; out float32 [T, H, P]; vectors dt_bias, a_log, skip [H] of w_dt
// (skip may be null); dt_raw of type dt_dt.
GFB_API int gfb_ssd_scan(const float* x, int ldx, int b_off, int c_off, const void* dt_raw, int dt_dt, int ld_dt, int dt_off,
                         const void* dt_bias, const void* a_log, const void* skip, int w_dt, float* state, long state_ld,
                         float* out, const int* cu_seqlens, const int* tok_seq, const int* slots, const int* lengths,
                         int n_seqs, int n_tokens, int H, int P, int N, int G, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (G <= 0 || H % G) return gfb_fail("gfb_ssd_scan: %d heads do not divide into %d groups", H, G);
    int RG = 0;
    const int rpt = pick_rpt(N, &RG, (long)n_seqs * H >= 512);
    if (!rpt) return gfb_fail("gfb_ssd_scan: a state of %d rows per head does not fit a warp", N);
    const int CB = SCAN_WARPS * (32 / RG);
    const unsigned slices = (unsigned)((P + CB - 1) / CB);
    if (H > 65535 || slices > 65535) return gfb_fail("gfb_ssd_scan: %d heads of %d columns exceed the grid limit", H, P);
    const size_t smem = ((size_t)2 * TB * (2 * RG * (rpt + ROW_PAD) + CB + 2) + (size_t)TB * CB) * sizeof(float);
    GfbBatch b{cu_seqlens, tok_seq, slots, lengths, n_seqs, n_tokens};
    cudaError_t e = cudaSuccess;
#define GO(TD, R)                                                                                                          \
    do {                                                                                                                   \
        if (allow_smem(ssd_scan_kernel<TD, R>, smem, "gfb_ssd_scan")) return 1;                                            \
        e = gfb_launch(ssd_scan_kernel<TD, R>, dim3(n_seqs, H, slices), dim3(32 * SCAN_WARPS), smem, stream, x, ldx, b_off, c_off, \
                       (const TD*)dt_raw, ld_dt, dt_off, dt_bias, a_log, skip, w_dt, state, (size_t)state_ld, out, b, H, P, N, G, RG); \
    } while (0)
#define PICK(TD) do { if (rpt == 8) GO(TD, 8); else if (rpt == 16) GO(TD, 16); else if (rpt == 32) GO(TD, 32); else GO(TD, 64); } while (0)
    if (dt_dt == GFB_BF16) PICK(__nv_bfloat16);
    else if (dt_dt == GFB_F32) PICK(float);
    else return gfb_fail("gfb_ssd_scan: unknown type %d", dt_dt);
#undef PICK
#undef GO
    return gfb_check(e, "gfb_ssd_scan");
}

// state float32: slot stride state_ld, per slot [H][d][dv]; out float32 [T, H, dv]; dt_bias [H * d], a_log [H] of w_dt.
// head_decay: one decay per head and token instead of one per key channel: a_raw has H columns from a_off, dt_bias is [H].
// qkv and a_raw are scratch of the caller: q and k are overwritten by their unit vectors, the decay inputs by the decays.
GFB_API int gfb_delta_rule(float* qkv, int ldq, int q_off, int k_off, int v_off, const void* beta_raw, int b_dt, int ld_b,
                           int beta_off, float* a_raw, int ld_a, int a_off, const void* dt_bias, const void* a_log, int w_dt,
                           float* state, long state_ld, float* out, const int* cu_seqlens, const int* tok_seq, const int* slots,
                           const int* lengths, int n_seqs, int n_tokens, int H, int KH, int d, int dv, float q_scale,
                           float unit_eps, int head_decay, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (KH <= 0 || H % KH) return gfb_fail("gfb_delta_rule: %d heads do not divide into %d query/key heads", H, KH);
    int RG = 0;
    const int rpt = pick_rpt(d, &RG, (long)n_seqs * H >= 512);
    if (!rpt) return gfb_fail("gfb_delta_rule: a state of %d rows per head does not fit a warp", d);
    const int CB = SCAN_WARPS * (32 / RG);
    const unsigned slices = (unsigned)((dv + CB - 1) / CB);
    if (H > 65535 || slices > 65535) return gfb_fail("gfb_delta_rule: %d heads of %d columns exceed the grid limit", H, dv);
    const size_t smem = ((size_t)2 * TB * (3 * RG * (rpt + ROW_PAD) + CB + 1) + (size_t)TB * CB * RG) * sizeof(float);
    GfbBatch b{cu_seqlens, tok_seq, slots, lengths, n_seqs, n_tokens};
    cudaError_t e = gfb_launch(delta_prepare_kernel, dim3(n_tokens), dim3(128), 0, stream, qkv, ldq, q_off, k_off, a_raw, ld_a, a_off,
                               dt_bias, a_log, w_dt, H, KH, d, q_scale, unit_eps, head_decay);
    if (gfb_check(e, "gfb_delta_rule (prepare)")) return 1;
#define GO(TD, R)                                                                                                          \
    do {                                                                                                                   \
        if (allow_smem(delta_rule_kernel<TD, R>, smem, "gfb_delta_rule")) return 1;                                        \
        e = gfb_launch(delta_rule_kernel<TD, R>, dim3(n_seqs, H, slices), dim3(32 * SCAN_WARPS), smem, stream, (const float*)qkv, ldq, \
                       q_off, k_off, v_off, (const TD*)beta_raw, ld_b, beta_off, (const float*)a_raw, ld_a, a_off, state,  \
                       (size_t)state_ld, out, b, H, KH, d, dv, RG, head_decay);                                            \
    } while (0)
#define PICK(TD) do { if (rpt == 8) GO(TD, 8); else if (rpt == 16) GO(TD, 16); else if (rpt == 32) GO(TD, 32); else GO(TD, 64); } while (0)
    if (b_dt == GFB_BF16) PICK(__nv_bfloat16);
    else if (b_dt == GFB_F32) PICK(float);
    else return gfb_fail("gfb_delta_rule: unknown type %d", b_dt);
#undef PICK
#undef GO
    return gfb_check(e, "gfb_delta_rule");
}

// ------------------------------------------------------------------------------ gated group norm ----
// One warp per (token, group of `gs` columns), or one block for a large group (BLOCK): v = y, times act(gate) first if
// gate_first; n = v / sqrt(mean(v^2) + eps) * weight[col % w_len]; times act(gate) behind the norm otherwise.
// act: 0 = SiLU, 1 = sigmoid.
template <typename TG, typename TO, bool BLOCK>
__global__ void gated_norm_kernel(const float* __restrict__ y, const TG* __restrict__ gate, int ld_gate, int gate_off,
                                  const void* __restrict__ weight, int w_dt, int w_len, TO* __restrict__ out, int T, int groups,
                                  int gs, float eps, int act, int gate_first) {
    __shared__ float scratch[32];
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int lane = BLOCK ? threadIdx.x : (threadIdx.x & 31), step = BLOCK ? blockDim.x : 32;
    const long item = BLOCK ? (long)blockIdx.x : (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long)T * groups) return;
    const int t = (int)(item / groups), g = (int)(item - (long)t * groups);
    const float* yr = y + ((size_t)t * groups + g) * gs;
    const TG* gr = gate + (size_t)t * ld_gate + gate_off + (size_t)g * gs;
    float ss = 0.f;
    for (int c = lane; c < gs; c += step) {
        float v = yr[c];
        if (gate_first) { const float z = gfb_to_f32(gr[c]); v *= act ? sigmoid_f(z) : silu_f(z); }
        ss = fmaf(v, v, ss);
    }
    ss = BLOCK ? gfb_block_sum(ss, scratch) : gfb_warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / (float)gs + eps);
    TO* o = out + ((size_t)t * groups + g) * gs;
    for (int c = lane; c < gs; c += step) {
        float v = yr[c];
        const float z = gfb_to_f32(gr[c]);
        const float a = act ? sigmoid_f(z) : silu_f(z);
        if (gate_first) v *= a;
        v = v * r * ldw(weight, w_dt, (size_t)(g * gs + c) % w_len);
        if (!gate_first) v *= a;
        o[c] = gfb_from_f32<TO>(v);
    }
}

// y float32 [T, groups * gs]; gate [T, ld_gate] of gate_dt, its groups * gs columns from gate_off; weight [w_len] of
// w_dt, indexed by column mod w_len; out [T, groups * gs] of out_dt.
GFB_API int gfb_gated_norm(const float* y, const void* gate, int gate_dt, int ld_gate, int gate_off, const void* weight, int w_dt,
                           int w_len, void* out, int out_dt, int T, int groups, int gs, float eps, int act, int gate_first,
                           cudaStream_t stream) {
    if (T <= 0 || groups <= 0 || gs <= 0) return 0;
    if (w_len <= 0) return gfb_fail("gfb_gated_norm: a weight of %d numbers", w_len);
    const long items = (long)T * groups;
    const bool big = gs > 512;                                  // a block per group instead of a warp
    const unsigned blocks = big ? (unsigned)items : (unsigned)((items + 3) / 4);
    const unsigned threads = big ? 256 : 128;
    typedef __nv_bfloat16 bf16;
    cudaError_t e;
#define GO(TG, TO)                                                                                                                \
    do {                                                                                                                          \
        if (big) e = gfb_launch(gated_norm_kernel<TG, TO, true>, dim3(blocks), dim3(threads), 0, stream, y, (const TG*)gate, ld_gate, \
                                gate_off, weight, w_dt, w_len, (TO*)out, T, groups, gs, eps, act, gate_first);                    \
        else e = gfb_launch(gated_norm_kernel<TG, TO, false>, dim3(blocks), dim3(threads), 0, stream, y, (const TG*)gate, ld_gate,    \
                            gate_off, weight, w_dt, w_len, (TO*)out, T, groups, gs, eps, act, gate_first);                        \
    } while (0)
    if (gate_dt == GFB_BF16 && out_dt == GFB_BF16) GO(bf16, bf16);
    else if (gate_dt == GFB_F32 && out_dt == GFB_BF16) GO(float, bf16);
    else if (gate_dt == GFB_F32 && out_dt == GFB_F32) GO(float, float);
    else if (gate_dt == GFB_BF16 && out_dt == GFB_F32) GO(bf16, float);
    else return gfb_fail("gfb_gated_norm: unsupported types gate %d out %d", gate_dt, out_dt);
#undef GO
    return gfb_check(e, "gfb_gated_norm");
}

// ------------------------------------------------------------------------------ gated linear recurrence ----
// Two kernels.  The gates of all tokens at once: a block takes a tile of RG_TOKENS tokens of one channel block, stages their
// inputs in shared memory (transposed, so that a thread reads four tokens of one input with one load) and each thread owns one
// output channel of the block for both gates: per input one weight of each gate (the matrices are stored [block][in][out], so a
// warp reads consecutive outputs) against the tile's tokens.  It leaves a and b = sqrt(1 - a^2) i u per token and channel.
// Then the recurrence: a thread per (sequence, channel) walks through the sequence's tokens of this step, S <- a S + b, and writes
// S gelu_tanh(y + by); a step with more than 64 tokens of a sequence walks in chunks side by side (below).
constexpr int RG_TOKENS = 16;
constexpr int RG_THREADS = 128;

__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
}

template <typename TW>
__global__ void __launch_bounds__(RG_THREADS)
rglru_gates_kernel(const float* __restrict__ u, const TW* __restrict__ wa, const TW* __restrict__ wi, const void* __restrict__ ba,
                   const void* __restrict__ bi, const void* __restrict__ lam, int v_dt, float decay_scale, float* __restrict__ a_out,
                   float* __restrict__ b_out, int T, int C, int bw) {
    extern __shared__ __align__(16) float us[];          // [bw][RG_TOKENS]
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int t0 = blockIdx.x * RG_TOKENS, blk = blockIdx.y;
    const int o = blockIdx.z * RG_THREADS + threadIdx.x;
    const int nt = min(RG_TOKENS, T - t0);
    for (int e = threadIdx.x; e < bw * RG_TOKENS; e += RG_THREADS) {
        const int tt = e / bw, i = e - tt * bw;         // consecutive threads read consecutive inputs of one token
        us[i * RG_TOKENS + tt] = tt < nt ? u[(size_t)(t0 + tt) * C + blk * bw + i] : 0.f;
    }
    __syncthreads();
    if (o >= bw) return;
    float ra[RG_TOKENS], ri[RG_TOKENS];
#pragma unroll
    for (int k = 0; k < RG_TOKENS; k++) ra[k] = ri[k] = 0.f;
    const TW* pa = wa + (size_t)blk * bw * bw + o;
    const TW* pi = wi + (size_t)blk * bw * bw + o;
#pragma unroll 4
    for (int i = 0; i < bw; i++) {
        const float xa = gfb_to_f32(pa[(size_t)i * bw]), xi = gfb_to_f32(pi[(size_t)i * bw]);
        const float4* row = reinterpret_cast<const float4*>(us + i * RG_TOKENS);
#pragma unroll
        for (int k4 = 0; k4 < RG_TOKENS / 4; k4++) {
            const float4 v = row[k4];
            ra[4 * k4 + 0] = fmaf(xa, v.x, ra[4 * k4 + 0]); ri[4 * k4 + 0] = fmaf(xi, v.x, ri[4 * k4 + 0]);
            ra[4 * k4 + 1] = fmaf(xa, v.y, ra[4 * k4 + 1]); ri[4 * k4 + 1] = fmaf(xi, v.y, ri[4 * k4 + 1]);
            ra[4 * k4 + 2] = fmaf(xa, v.z, ra[4 * k4 + 2]); ri[4 * k4 + 2] = fmaf(xi, v.z, ri[4 * k4 + 2]);
            ra[4 * k4 + 3] = fmaf(xa, v.w, ra[4 * k4 + 3]); ri[4 * k4 + 3] = fmaf(xi, v.w, ri[4 * k4 + 3]);
        }
    }
    const int c = blk * bw + o;
    const float bias_a = ldw(ba, v_dt, c), bias_i = ldw(bi, v_dt, c);
    const float rate = decay_scale * softplus_f(ldw(lam, v_dt, c));
#pragma unroll
    for (int k = 0; k < RG_TOKENS; k++) {
        if (k < nt) {
            const float r = sigmoid_f(ra[k] + bias_a), g = sigmoid_f(ri[k] + bias_i);
            const float log_a = -rate * r;
            const size_t at = (size_t)(t0 + k) * C + c;
            a_out[at] = expf(log_a);
            b_out[at] = sqrtf(-expm1f(2.0f * log_a)) * g * us[o * RG_TOKENS + k];
        }
    }
}

template <typename TY, typename TO>
__global__ void __launch_bounds__(RG_THREADS)
rglru_scan_kernel(const float* __restrict__ a, const float* __restrict__ bb, const TY* __restrict__ y, int ld_y, int y_off,
                  const void* __restrict__ y_bias, int v_dt, float* __restrict__ state, size_t state_ld, TO* __restrict__ out,
                  GfbBatch b, int C) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int s = blockIdx.x;
    const int c = blockIdx.y * RG_THREADS + threadIdx.x;
    if (c >= C) return;
    const int t0 = b.cu_seqlens[s], n = b.cu_seqlens[s + 1] - t0;
    float* st = state + (size_t)b.slots[s] * state_ld + c;
    const float yb = y_bias != nullptr ? ldw(y_bias, v_dt, c) : 0.f;
    float S = *st;
    constexpr int U = 8;
    for (int i0 = 0; i0 < n; i0 += U) {
        float av[U], bv[U], yv[U];
#pragma unroll
        for (int k = 0; k < U; k++) {
            const int t = t0 + min(i0 + k, n - 1);
            av[k] = a[(size_t)t * C + c];
            bv[k] = bb[(size_t)t * C + c];
            yv[k] = gfb_to_f32(y[(size_t)t * ld_y + y_off + c]);
        }
#pragma unroll
        for (int k = 0; k < U; k++) {
            if (i0 + k < n) {
                S = fmaf(av[k], S, bv[k]);
                out[(size_t)(t0 + i0 + k) * C + c] = gfb_from_f32<TO>(S * gelu_tanh_f(yv[k] + yb));
            }
        }
    }
    *st = S;
}

// Prompts: the same recurrence in chunks of RG_CHUNK tokens, which all run side by side.  S <- a S + b is a composition of
// affine maps, so a chunk is summed up as (P, Q) = (product of its a, its end state from zero); a short walk over a sequence's
// chunks gives every chunk the state it starts from (and the sequence its new state); then every chunk walks its tokens from there.
constexpr int RG_CHUNK = 64;

__global__ void __launch_bounds__(RG_THREADS)
rglru_chunk_kernel(const float* __restrict__ a, const float* __restrict__ bb, float* __restrict__ P, float* __restrict__ Q, GfbBatch b,
                   int C, int max_chunks) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int s = blockIdx.x, k = blockIdx.y;
    const int c = blockIdx.z * RG_THREADS + threadIdx.x;
    const int t0 = b.cu_seqlens[s], n = b.cu_seqlens[s + 1] - t0;
    if (c >= C || k * RG_CHUNK >= n) return;
    const int first = t0 + k * RG_CHUNK, count = min(RG_CHUNK, n - k * RG_CHUNK);
    float prod = 1.f, end = 0.f;
    constexpr int U = 8;
    for (int i0 = 0; i0 < count; i0 += U) {
        float av[U], bv[U];
#pragma unroll
        for (int j = 0; j < U; j++) {
            const int t = first + min(i0 + j, count - 1);
            av[j] = a[(size_t)t * C + c];
            bv[j] = bb[(size_t)t * C + c];
        }
#pragma unroll
        for (int j = 0; j < U; j++)
            if (i0 + j < count) { prod *= av[j]; end = fmaf(av[j], end, bv[j]); }
    }
    const size_t at = ((size_t)s * max_chunks + k) * C + c;
    P[at] = prod;
    Q[at] = end;
}

// P is overwritten by the state every chunk starts from
__global__ void __launch_bounds__(RG_THREADS)
rglru_carry_kernel(float* __restrict__ P, const float* __restrict__ Q, float* __restrict__ state, size_t state_ld, GfbBatch b, int C,
                   int max_chunks) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int s = blockIdx.x;
    const int c = blockIdx.y * RG_THREADS + threadIdx.x;
    if (c >= C) return;
    const int n = b.cu_seqlens[s + 1] - b.cu_seqlens[s];
    const int chunks = (n + RG_CHUNK - 1) / RG_CHUNK;
    float* st = state + (size_t)b.slots[s] * state_ld + c;
    float S = *st;
    for (int k = 0; k < chunks; k++) {
        const size_t at = ((size_t)s * max_chunks + k) * C + c;
        const float p = P[at];
        P[at] = S;
        S = fmaf(p, S, Q[at]);
    }
    *st = S;
}

template <typename TY, typename TO>
__global__ void __launch_bounds__(RG_THREADS)
rglru_apply_kernel(const float* __restrict__ a, const float* __restrict__ bb, const float* __restrict__ start, const TY* __restrict__ y,
                   int ld_y, int y_off, const void* __restrict__ y_bias, int v_dt, TO* __restrict__ out, GfbBatch b, int C, int max_chunks) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int s = blockIdx.x, k = blockIdx.y;
    const int c = blockIdx.z * RG_THREADS + threadIdx.x;
    const int t0 = b.cu_seqlens[s], n = b.cu_seqlens[s + 1] - t0;
    if (c >= C || k * RG_CHUNK >= n) return;
    const int first = t0 + k * RG_CHUNK, count = min(RG_CHUNK, n - k * RG_CHUNK);
    const float yb = y_bias != nullptr ? ldw(y_bias, v_dt, c) : 0.f;
    float S = start[((size_t)s * max_chunks + k) * C + c];
    constexpr int U = 8;
    for (int i0 = 0; i0 < count; i0 += U) {
        float av[U], bv[U], yv[U];
#pragma unroll
        for (int j = 0; j < U; j++) {
            const int t = first + min(i0 + j, count - 1);
            av[j] = a[(size_t)t * C + c];
            bv[j] = bb[(size_t)t * C + c];
            yv[j] = gfb_to_f32(y[(size_t)t * ld_y + y_off + c]);
        }
#pragma unroll
        for (int j = 0; j < U; j++)
            if (i0 + j < count) {
                S = fmaf(av[j], S, bv[j]);
                out[(size_t)(first + i0 + j) * C + c] = gfb_from_f32<TO>(S * gelu_tanh_f(yv[j] + yb));
            }
    }
}

// u float32 [T, C]: the recurrence's inputs.  wa, wi [blocks][C / blocks (in)][C / blocks (out)] of type w_dt: the two gates'
// matrices, transposed per block.  ba, bi, lam, y_bias [C] of type v_dt.  y [T, ld_y] of type y_dt, its C columns from y_off.
// state float32, slot stride state_ld, C numbers per slot.  out [T, C] of type out_dt.  scratch float32 [2][T][C], and behind it,
// where the longest sequence of the step (max_q_len) has more than one chunk of 64 tokens, [2][n_seqs][chunks of max_q_len][C].
GFB_API long gfb_rglru_scratch_floats(int n_tokens, int n_seqs, int max_q_len, int C) {
    long need = 2L * n_tokens * C;
    if (max_q_len > RG_CHUNK) need += 2L * n_seqs * ((max_q_len + RG_CHUNK - 1) / RG_CHUNK) * C;
    return need;
}

GFB_API int gfb_rglru(const float* u, const void* wa, const void* wi, int w_dt, const void* ba, const void* bi, const void* lam,
                      const void* y_bias, int v_dt, float decay_scale, const void* y, int y_dt, int ld_y, int y_off, float* state,
                      long state_ld, void* out, int out_dt, float* scratch, const int* cu_seqlens, const int* tok_seq, const int* slots,
                      const int* lengths, int n_seqs, int n_tokens, int max_q_len, int C, int blocks, cudaStream_t stream) {
    if (n_tokens <= 0 || C <= 0) return 0;
    if (blocks < 1 || C % blocks) return gfb_fail("gfb_rglru: %d channels do not divide into %d blocks", C, blocks);
    const int bw = C / blocks;
    const size_t smem = (size_t)bw * RG_TOKENS * sizeof(float);
    if (smem > 200 * 1024) return gfb_fail("gfb_rglru: blocks of %d channels exceed the kernel's shared memory", bw);
    if (blocks > 65535 || (bw + RG_THREADS - 1) / RG_THREADS > 65535) return gfb_fail("gfb_rglru: too many blocks");
    GfbBatch b{cu_seqlens, tok_seq, slots, lengths, n_seqs, n_tokens};
    float* a_buf = scratch;
    float* b_buf = scratch + (size_t)n_tokens * C;
    const dim3 grid((n_tokens + RG_TOKENS - 1) / RG_TOKENS, blocks, (bw + RG_THREADS - 1) / RG_THREADS);
    cudaError_t e;
#define GATES(TW)                                                                                                              \
    do {                                                                                                                       \
        static size_t allowed = 48 * 1024;                                                                                     \
        if (smem > allowed) {                                                                                                  \
            cudaFuncSetAttribute(rglru_gates_kernel<TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);             \
            allowed = 200 * 1024;                                                                                              \
        }                                                                                                                      \
        e = gfb_launch(rglru_gates_kernel<TW>, grid, dim3(RG_THREADS), smem, stream, u, (const TW*)wa, (const TW*)wi, ba, bi, lam, \
                       v_dt, decay_scale, a_buf, b_buf, n_tokens, C, bw);                                                      \
    } while (0)
    if (w_dt == GFB_BF16) GATES(__nv_bfloat16);
    else if (w_dt == GFB_F32) GATES(float);
    else return gfb_fail("gfb_rglru: unknown weight type %d", w_dt);
#undef GATES
    if (gfb_check(e, "gfb_rglru (gates)")) return 1;
    const dim3 sgrid(n_seqs, (C + RG_THREADS - 1) / RG_THREADS);
    typedef __nv_bfloat16 bf16;
    if (max_q_len > RG_CHUNK) {
        const int max_chunks = (max_q_len + RG_CHUNK - 1) / RG_CHUNK;
        if (max_chunks > 65535) return gfb_fail("gfb_rglru: a step of %d tokens of one sequence", max_q_len);
        float* P = b_buf + (size_t)n_tokens * C;
        float* Q = P + (size_t)n_seqs * max_chunks * C;
        const dim3 cgrid(n_seqs, max_chunks, (C + RG_THREADS - 1) / RG_THREADS);
        e = gfb_launch(rglru_chunk_kernel, cgrid, dim3(RG_THREADS), 0, stream, (const float*)a_buf, (const float*)b_buf, P, Q, b, C, max_chunks);
        if (gfb_check(e, "gfb_rglru (chunks)")) return 1;
        e = gfb_launch(rglru_carry_kernel, sgrid, dim3(RG_THREADS), 0, stream, P, (const float*)Q, state, (size_t)state_ld, b, C, max_chunks);
        if (gfb_check(e, "gfb_rglru (carry)")) return 1;
#define APPLY(TY, TO) e = gfb_launch(rglru_apply_kernel<TY, TO>, cgrid, dim3(RG_THREADS), 0, stream, (const float*)a_buf, (const float*)b_buf, \
                                     (const float*)P, (const TY*)y, ld_y, y_off, y_bias, v_dt, (TO*)out, b, C, max_chunks)
        if (y_dt == GFB_BF16 && out_dt == GFB_BF16) APPLY(bf16, bf16);
        else if (y_dt == GFB_F32 && out_dt == GFB_F32) APPLY(float, float);
        else if (y_dt == GFB_F32 && out_dt == GFB_BF16) APPLY(float, bf16);
        else return gfb_fail("gfb_rglru: unsupported types y %d out %d", y_dt, out_dt);
#undef APPLY
        return gfb_check(e, "gfb_rglru (apply)");
    }
#define SCAN(TY, TO) e = gfb_launch(rglru_scan_kernel<TY, TO>, sgrid, dim3(RG_THREADS), 0, stream, (const float*)a_buf, (const float*)b_buf, \
                                    (const TY*)y, ld_y, y_off, y_bias, v_dt, state, (size_t)state_ld, (TO*)out, b, C)
    if (y_dt == GFB_BF16 && out_dt == GFB_BF16) SCAN(bf16, bf16);
    else if (y_dt == GFB_F32 && out_dt == GFB_F32) SCAN(float, float);
    else if (y_dt == GFB_F32 && out_dt == GFB_BF16) SCAN(float, bf16);
    else return gfb_fail("gfb_rglru: unsupported types y %d out %d", y_dt, out_dt);
#undef SCAN
    return gfb_check(e, "gfb_rglru (scan)");
}
