// What happens to q, k and v between their projection and the attention, for mixers that the
// rotate-and-append kernel of core.cu does not cover: any subset of
//   - per-head root-mean-square norm of q and of k with a weight shared by the heads
//     (v / sqrt(mean(v^2) + eps) * w, 32-bit), or the same norm over the whole projection
//     (all heads of q, or of k, as one vector, with a weight per column),
//   - rotation of the first rot_dims dimensions of each q and k head by the token's position
//     (pairs (2i, 2i+1) or (i, i + rot_dims/2); the other dimensions pass),
//   - a factor on k,
// and then q to q_out, k and v to the token's place in the paged cache.  Keys and values may have
// different head sizes (dk, dv).  The source row holds q, k and v at given offsets, in the model's
// type or as 32-bit partial sums of a product split over K.
// The per-head norm may come without a weight (NORM_BARE) and may run behind the rotation instead of ahead
// of it (NORM_LAST).  `maps` > 1: every query head and every key head is `maps` vectors of dk side by side
// (several score maps over one set of values); each is normed and rotated as a head of its own, and a cached
// key row holds the `maps` vectors of its head one after the other.
// One warp per (token, head); the head sits in shared memory between the steps.
#include "common.cuh"

GFB_DEFINE_LAST_ERROR()

constexpr int WARPS = 4;
enum { NORM_WHOLE = 1, NORM_BARE = 2, NORM_LAST = 4, Q_SPREAD = 8 };

__device__ __forceinline__ float ld_w(const void* p, int dt, int i) {
    return dt == GFB_BF16 ? __bfloat162float(((const __nv_bfloat16*)p)[i]) : ((const float*)p)[i];
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
qkv_prepare_kernel(const void* __restrict__ src, int S, size_t slice, int width, int q_off, int k_off, int v_off,
                   T* __restrict__ q_out, GfbPagedKV kv, GfbBatch b, const float* __restrict__ table, int table_len,
                   int rot_dims, int pairing, const void* q_norm, const void* k_norm, int w_dt, float eps, float k_scale,
                   int H, int GK, int G, int maps, int dk, int dv, int dmax, int append, int norm_opts, int* status) {
    extern __shared__ float heads[];
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int per_token = H + (append ? GK + G : 0);
    const int norm_whole = norm_opts & NORM_WHOLE;
    const long item = (long)blockIdx.x * WARPS + warp;
    if (item >= (long)b.n_tokens * per_token) return;
    const int t = (int)(item / per_token), head = (int)(item - (long)t * per_token);
    float* v = heads + (size_t)warp * dmax;
    const int s = b.tok_seq[t];
    const int slot = b.slots[s];
    const int pos = b.lengths[slot] + (t - b.cu_seqlens[s]);
    const bool is_q = head < H, is_k = !is_q && head < H + GK;
    const int d = (is_q || is_k) ? dk : dv;
    bool ok = pos >= 0 && (table == nullptr || pos < table_len);
    T* dst = nullptr;
    if (is_q) {
        // Q_SPREAD: q_out rows are maps * dk wide and map m of a head sits at columns m * dk .. of its own row (the rest stays
        // as the caller left it: zeros), so that against a cached row of `maps` keys side by side it meets its own key only
        dst = (norm_opts & Q_SPREAD) ? q_out + (((size_t)t * H + head) * maps + head % maps) * dk : q_out + ((size_t)t * H + head) * dk;
    } else {
        const int pi = pos / kv.page_size, off = pos - pi * kv.page_size;
        const int page = (ok && pi < kv.max_pages) ? kv.page_table[(size_t)slot * kv.max_pages + pi] : -1;
        if (page < 0 || page >= kv.n_pages) ok = false;
        else if (is_k) dst = (T*)kv.k_pool + (((size_t)page * G + (head - H) / maps) * kv.page_size + off) * ((size_t)dk * maps)
                             + (size_t)((head - H) % maps) * dk;
        else dst = (T*)kv.v_pool + (((size_t)page * G + (head - H - GK)) * kv.page_size + off) * dv;
    }
    if (!ok) {
        if (lane == 0 && head == 0) gfb_report(status, GFB_ERR_CACHE_RANGE, t, pos);
        if (is_q) for (int i = lane; i < dk; i += 32) dst[i] = gfb_from_f32<T>(0.f);     // q stays defined
        return;
    }
    const size_t e0 = (size_t)t * width + (is_q ? q_off + head * dk : is_k ? k_off + (head - H) * dk : v_off + (head - H - GK) * dv);
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) {
        float x;
        if (S > 0) {
            const float* p = (const float*)src;
            x = 0.f;
            for (int k = 0; k < S; k++) x += p[(size_t)k * slice + e0 + i];
        } else {
            x = gfb_to_f32(((const T*)src)[e0 + i]);
        }
        v[i] = x;
        ss += x * x;
    }
    const void* nw = is_q ? q_norm : is_k ? k_norm : nullptr;
    if (nw != nullptr && norm_whole) {
        // the statistic spans every head of the projection; each head's warp adds it up for itself, in the same order
        const int heads = is_q ? H : GK, local = is_q ? head : head - H;
        const size_t p0 = (size_t)t * width + (is_q ? q_off : k_off);
        float tot = 0.f;
        for (int i = lane; i < heads * dk; i += 32) {
            float x;
            if (S > 0) {
                const float* p = (const float*)src;
                x = 0.f;
                for (int k = 0; k < S; k++) x += p[(size_t)k * slice + p0 + i];
            } else {
                x = gfb_to_f32(((const T*)src)[p0 + i]);
            }
            tot += x * x;
        }
        tot = gfb_warp_sum(tot);
        const float r = 1.0f / sqrtf(tot / (float)(heads * dk) + eps);
        for (int i = lane; i < d; i += 32) v[i] = v[i] * r * ld_w(nw, w_dt, local * dk + i);
    } else if ((is_q || is_k) && (nw != nullptr || (norm_opts & NORM_BARE)) && !(norm_opts & NORM_LAST)) {
        ss = gfb_warp_sum(ss);
        const float r = 1.0f / sqrtf(ss / (float)d + eps);
        for (int i = lane; i < d; i += 32) v[i] = v[i] * r * (nw != nullptr ? ld_w(nw, w_dt, i) : 1.f);
    }
    __syncwarp();
    const float f = is_k ? k_scale : 1.f;
    if (table != nullptr && (is_q || is_k)) {
        const int half = rot_dims >> 1;
        const float* cs = table + (size_t)pos * half * 2;
        for (int i = lane; i < half; i += 32) {
            const int i0 = pairing == 1 ? i : 2 * i, i1 = pairing == 1 ? i + half : 2 * i + 1;
            const float c = cs[2 * i], sn = cs[2 * i + 1], a = v[i0], bb = v[i1];
            v[i0] = a * c - bb * sn;
            v[i1] = bb * c + a * sn;
        }
        __syncwarp();
    }
    if ((is_q || is_k) && (norm_opts & NORM_LAST) && !norm_whole && (nw != nullptr || (norm_opts & NORM_BARE))) {
        float s2 = 0.f;
        for (int i = lane; i < d; i += 32) s2 += v[i] * v[i];
        s2 = gfb_warp_sum(s2);
        const float r = 1.0f / sqrtf(s2 / (float)d + eps);
        for (int i = lane; i < d; i += 32) v[i] = v[i] * r * (nw != nullptr ? ld_w(nw, w_dt, i) : 1.f);
    }
    for (int i = lane; i < d; i += 32) dst[i] = gfb_from_f32<T>(v[i] * f);
}

// src: [T, width] of type dt, or with n_partials > 0 float32 [n_partials][T][width]; q at q_off (H heads of dk), k at
// k_off (G heads of dk), v at v_off (G heads of dv).  table (or null: no rotation): float32 [table_len][rot_dims/2][2].
// q_norm / k_norm (or null): [dk] of type w_dt, or with NORM_WHOLE [H * dk] and [G * dk].  append = 0: only q is produced.
// norm_opts: NORM_WHOLE | NORM_BARE (a per-head norm also where no weight is given) | NORM_LAST (the per-head norm follows
// the rotation) | Q_SPREAD (q_out is [T, H * maps, maps * dk], zeroed by the caller; query j is written at columns
// (j mod maps) * dk of row j).  maps >= 1: H and G count heads; q_out is [T, H * maps, dk], key rows of the cache hold maps * dk numbers.
GFB_API int gfb_qkv_prepare(const void* src, int n_partials, int width, int q_off, int k_off, int v_off, void* q_out, int dt,
                            void* k_pool, void* v_pool, const int* page_table, int max_pages, int page_size, int n_pages,
                            const int* cu_seqlens, const int* tok_seq, const int* slots, const int* lengths, int n_seqs,
                            int n_tokens, const float* table, int table_len, int rot_dims, int pairing,
                            const void* q_norm, const void* k_norm, int w_dt, float eps, float k_scale,
                            int H, int G, int dk, int dv, int append, int norm_opts, int maps, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (maps < 1) return gfb_fail("gfb_qkv_prepare: %d score maps per head", maps);
    const int HQ = H * maps, GK = G * maps;
    if (table != nullptr && (rot_dims % 2 || rot_dims > dk || rot_dims < 0))
        return gfb_fail("gfb_qkv_prepare: %d rotated dimensions in a head of %d", rot_dims, dk);
    GfbPagedKV kv{k_pool, v_pool, page_table, max_pages, page_size, n_pages};
    GfbBatch b{cu_seqlens, tok_seq, slots, lengths, n_seqs, n_tokens};
    const int dmax = dk > dv ? dk : dv;
    const long items = (long)n_tokens * (HQ + (append ? GK + G : 0));
    const long blocks = (items + WARPS - 1) / WARPS;
    if (blocks > 0x7fffffffL) return gfb_fail("gfb_qkv_prepare: too many heads");
    const size_t smem = (size_t)WARPS * dmax * sizeof(float);
    if (smem > 48 * 1024) return gfb_fail("gfb_qkv_prepare: heads of %d exceed the kernel's shared memory", dmax);
    const size_t slice = (size_t)n_tokens * width;
    cudaError_t e;
#define GO(T) e = gfb_launch(qkv_prepare_kernel<T>, dim3((unsigned)blocks), dim3(WARPS * 32), smem, stream, src, n_partials, slice, \
                             width, q_off, k_off, v_off, (T*)q_out, kv, b, table, table_len, rot_dims, pairing, q_norm, k_norm, \
                             w_dt, eps, k_scale, HQ, GK, G, maps, dk, dv, dmax, append, norm_opts, status)
    if (dt == GFB_BF16) GO(__nv_bfloat16);
    else if (dt == GFB_F32) GO(float);
    else return gfb_fail("gfb_qkv_prepare: unknown type %d", dt);
#undef GO
    return gfb_check(e, "gfb_qkv_prepare");
}
