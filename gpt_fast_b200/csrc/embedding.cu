// Token embedding plus a hashed bigram embedding:
//
//     out[t] = table[tok_t] * scale + extra[(tok_(t-1) * mul_prev + tok_t * mul_cur) mod buckets]
//
// with row `buckets` of `extra` (its last row) for the first token of a sequence.  The token before a
// step's first token is per-sequence state: prev[slot], written by a second small kernel behind the
// first (the last token of every sequence of the step), so that a sequence may arrive in any portions.
// The sum is 32-bit.
//
// And token embedding plus a learned vector per position: out[t] = table[tok_t] * scale + positions[p_t], p_t the
// token's place in its sequence.
#include "common.cuh"

GFB_DEFINE_LAST_ERROR()

template <typename TW>
__global__ void embed_hashed_kernel(const int* __restrict__ tokens, const TW* __restrict__ table, const TW* __restrict__ extra,
                                    float* __restrict__ out, GfbBatch b, const int* __restrict__ prev, int D, int V,
                                    int buckets, long long mul_prev, long long mul_cur, float scale, int* status) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int t = blockIdx.x;
    const int id = tokens[t];
    float* o = out + (size_t)t * D;
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0) gfb_report(status, GFB_ERR_TOKEN_RANGE, t, id);
        for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const int s = b.tok_seq[t];
    const int slot = b.slots[s];
    long long row = buckets;                                  // a sequence's first token
    int before = -1;
    if (t > b.cu_seqlens[s]) before = tokens[t - 1];
    else if (b.lengths[slot] > 0) before = prev[slot];
    if (before >= 0) {
        row = ((long long)before * mul_prev + (long long)id * mul_cur) % buckets;      // 64-bit: the multipliers may be large
        if (row < 0) row += buckets;
    }
    const TW* e = table + (size_t)id * D;
    const TW* x = extra + (size_t)row * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = gfb_to_f32(e[i]) * scale + gfb_to_f32(x[i]);
}

__global__ void embed_prev_kernel(const int* __restrict__ tokens, GfbBatch b, int* __restrict__ prev) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= b.n_seqs) return;
    const int end = b.cu_seqlens[s + 1];
    if (end > b.cu_seqlens[s]) prev[b.slots[s]] = tokens[end - 1];
}

// tokens int32 [T]; table [V, D] and extra [buckets + 1, D] of type table_dt; out float32 [T, D]; prev int32 [n_slots].
GFB_API int gfb_embed_hashed(const int* tokens, const void* table, const void* extra, int table_dt, float* out,
                             const int* cu_seqlens, const int* tok_seq, const int* slots, const int* lengths, int n_seqs,
                             int n_tokens, int* prev, int D, int V, int buckets, long long mul_prev, long long mul_cur, float scale,
                             int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (buckets <= 0) return gfb_fail("gfb_embed_hashed: %d buckets", buckets);
    GfbBatch b{cu_seqlens, tok_seq, slots, lengths, n_seqs, n_tokens};
    const int threads = D >= 1024 ? 256 : 128;
    cudaError_t e;
    if (table_dt == GFB_BF16)
        e = gfb_launch(embed_hashed_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, stream, tokens, (const __nv_bfloat16*)table,
                       (const __nv_bfloat16*)extra, out, b, (const int*)prev, D, V, buckets, mul_prev, mul_cur, scale, status);
    else if (table_dt == GFB_F32)
        e = gfb_launch(embed_hashed_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, tokens, (const float*)table,
                       (const float*)extra, out, b, (const int*)prev, D, V, buckets, mul_prev, mul_cur, scale, status);
    else
        return gfb_fail("gfb_embed_hashed: unknown table type %d", table_dt);
    if (gfb_check(e, "gfb_embed_hashed")) return 1;
    e = gfb_launch(embed_prev_kernel, dim3((n_seqs + 127) / 128), dim3(128), 0, stream, tokens, b, prev);
    return gfb_check(e, "gfb_embed_hashed (previous token)");
}

template <typename TW>
__global__ void embed_positions_kernel(const int* __restrict__ tokens, const TW* __restrict__ table, const TW* __restrict__ positions,
                                       float* __restrict__ out, GfbBatch b, int D, int V, int P, float scale, int* status) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int t = blockIdx.x;
    const int id = tokens[t];
    const int s = b.tok_seq[t];
    const int pos = b.lengths[b.slots[s]] + (t - b.cu_seqlens[s]);
    float* o = out + (size_t)t * D;
    const bool bad_id = id < 0 || id >= V, bad_pos = pos < 0 || pos >= P;
    if (bad_id || bad_pos) {
        if (threadIdx.x == 0) {
            if (bad_id) gfb_report(status, GFB_ERR_TOKEN_RANGE, t, id);
            else gfb_report(status, GFB_ERR_CACHE_RANGE, t, pos);
        }
        for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const TW* e = table + (size_t)id * D;
    const TW* x = positions + (size_t)pos * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = gfb_to_f32(e[i]) * scale + gfb_to_f32(x[i]);
}

// tokens int32 [T]; table [V, D] and positions [P, D] of type table_dt; out float32 [T, D].
GFB_API int gfb_embed_positions(const int* tokens, const void* table, const void* positions, int table_dt, float* out,
                                const int* cu_seqlens, const int* tok_seq, const int* slots, const int* lengths, int n_seqs,
                                int n_tokens, int D, int V, int P, float scale, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    GfbBatch b{cu_seqlens, tok_seq, slots, lengths, n_seqs, n_tokens};
    const int threads = D >= 1024 ? 256 : 128;
    cudaError_t e;
    if (table_dt == GFB_BF16)
        e = gfb_launch(embed_positions_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, stream, tokens, (const __nv_bfloat16*)table,
                       (const __nv_bfloat16*)positions, out, b, D, V, P, scale, status);
    else if (table_dt == GFB_F32)
        e = gfb_launch(embed_positions_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, tokens, (const float*)table,
                       (const float*)positions, out, b, D, V, P, scale, status);
    else
        return gfb_fail("gfb_embed_positions: unknown table type %d", table_dt);
    return gfb_check(e, "gfb_embed_positions");
}
