// Causal grouped-query attention over the paged cache, for any head size, any
// number of heads and groups, any mix of query lengths, both precisions.
//
// It stands where gpt-fast expands K/V to all heads and calls SDPA over the
// whole cache with a boolean mask (model.py:209-211): query head h reads
// key/value head h / (H/G); the key at position j is visible to the query at
// position p iff j <= p (and p - j < window when a window is set); scores are
// scaled by `scale`; softmax is 32-bit.  Options that other mixers use: `chunk` (a query
// sees only keys of its own block of `chunk` positions, blocks counted from
// position 0 of the sequence), `sink` (one number per query head whose
// exponential joins the softmax denominator without a value), a value head
// size `dv` of its own, values that are the leading part of the key rows, and a
// bias on the scaled score that depends on head and distance n = p - j only:
// `bias` (a table [bias_len][H], row min(n, bias_len - 1), added) and `slopes`
// (one number per head, slopes[h] * n taken off).  `softcap` > 0 squashes the (scaled, biased)
// score to cap * tanh(score / cap).  `keep_first`: the sequence's first keep_first positions stay
// visible to every later query whatever the window.  `maps` = 2: a head has two queries and a key
// row two keys side by side, each pair a softmax of its own over the same values; the head's output
// is o = o_1 - lambda o_2, divided by its root mean square over dv (diff_eps inside the root) and
// multiplied by out_scale.
//
// One block per (token, query head).  Keys are visited in chunks of 128 that
// start at multiples of 128 of the ABSOLUTE position, with an online softmax
// between chunks, so a query's result is the same bits whether its token came
// in a long prompt, alone, or in any batch.  This is the kernel of the 32-bit
// path and the fallback of the bfloat16 path; the fast bfloat16 kernels live
// in files of their own.
#include "common.cuh"

GFB_DEFINE_LAST_ERROR()

constexpr int CHUNK = 128;      // keys per step = threads per block
constexpr int MAX_DPT = 4;      // head_dim <= CHUNK * MAX_DPT

template <typename T>
__global__ void __launch_bounds__(CHUNK)
attention_generic_kernel(const T* __restrict__ q, T* __restrict__ out, GfbPagedKV kv, GfbBatch b,
                         int H, int G, int d, int dv, int v_row, float scale, int window, int chunk,
                         const float* __restrict__ sink, const float* __restrict__ bias, int bias_len,
                         const float* __restrict__ slopes, float softcap, int keep_first, int maps, float lambda,
                         float diff_eps, float out_scale, int* status) {
    extern __shared__ float smem[];
    float* qs = smem;              // [d]
    float* ps = smem + d;          // [CHUNK]
    __shared__ float scratch[32];
    __shared__ int page_of[CHUNK]; // page ids of the current chunk (2 pages of 64, or fewer larger ones)
    gfb_pdl_launch();
    gfb_pdl_wait();

    int t = blockIdx.x, h = blockIdx.y;
    int g = h / (H / G);
    int s = b.tok_seq[t];
    int slot = b.slots[s];
    int pos = b.lengths[slot] + (t - b.cu_seqlens[s]);
    const int dkr = d * maps;                    // numbers in a cached key row

    int lo = 0;
    if (window > 0 && pos - window + 1 > 0) lo = pos - window + 1;
    if (chunk > 0) lo = max(lo, (pos / chunk) * chunk);
    const int* pt = kv.page_table + (size_t)slot * kv.max_pages;
    const size_t head_off = (size_t)g * kv.page_size * dkr, v_head_off = (size_t)g * kv.page_size * v_row;
    const size_t page_stride = (size_t)G * kv.page_size * dkr, v_page_stride = (size_t)G * kv.page_size * v_row;
    const int kept = lo > 0 ? min(keep_first, lo) : 0;       // positions [0, kept) are seen besides [lo, pos]
    float first[MAX_DPT];                                    // the first map's finished output, while the second runs
#pragma unroll
    for (int i = 0; i < MAX_DPT; i++) first[i] = 0.f;

  for (int map = 0; map < maps; map++) {
    __syncthreads();               // every thread is done with the previous map's qs
    const T* qrow = q + (((size_t)t * H + h) * maps + map) * d;
    for (int i = threadIdx.x; i < d; i += CHUNK) qs[i] = gfb_to_f32(qrow[i]) * scale;
    float m_run = -INFINITY, l_run = 0.f;
    float acc[MAX_DPT];
#pragma unroll
    for (int i = 0; i < MAX_DPT; i++) acc[i] = 0.f;

    for (int c0 = kept > 0 ? 0 : (lo / CHUNK) * CHUNK; c0 <= pos; c0 += CHUNK) {
        if (c0 >= kept && c0 + CHUNK <= lo) continue;          // a block of keys between the kept ones and the window
        __syncthreads();           // qs ready (first pass); ps / page_of free (later passes)
        int j = c0 + threadIdx.x;
        bool live = (j >= lo || j < kept) && j <= pos;
        int page = -1;
        if (live) {
            int pi = j / kv.page_size;
            page = pi < kv.max_pages ? pt[pi] : -1;
            if (page < 0 || page >= kv.n_pages) {
                gfb_report(status, GFB_ERR_PAGE_TABLE, slot, pi);
                live = false;
                page = -1;
            }
        }
        page_of[threadIdx.x] = page;
        float sc = -INFINITY;
        if (live) {
            const T* krow = (const T*)kv.k_pool + (size_t)page * page_stride + head_off
                            + (size_t)(j % kv.page_size) * dkr + (size_t)map * d;
            float dot = 0.f;
            for (int i = 0; i < d; i++) dot = fmaf(qs[i], gfb_to_f32(krow[i]), dot);
            sc = dot;
            if (bias != nullptr) sc += bias[(size_t)min(pos - j, bias_len - 1) * H + h];
            if (slopes != nullptr) sc -= slopes[h] * (float)(pos - j);
            if (softcap > 0.f) sc = softcap * tanhf(sc / softcap);
        }
        float m_new = fmaxf(m_run, gfb_block_max(sc, scratch));
        float p = live ? expf(sc - m_new) : 0.f;
        ps[threadIdx.x] = p;
        float l_chunk = gfb_block_sum(p, scratch);     // also orders the ps / page_of stores
        float corr = (m_run == -INFINITY) ? 0.f : expf(m_run - m_new);
        l_run = l_run * corr + l_chunk;
        m_run = m_new;
        int nkeys = min(CHUNK, pos - c0 + 1);
#pragma unroll
        for (int r = 0; r < MAX_DPT; r++) {
            int dim = threadIdx.x + r * CHUNK;
            if (dim < dv) {
                float a = acc[r] * corr;
                for (int jj = 0; jj < nkeys; jj++) {
                    int pg = page_of[jj];
                    if (pg < 0) continue;
                    const T* vrow = (const T*)kv.v_pool + (size_t)pg * v_page_stride + v_head_off
                                    + (size_t)((c0 + jj) % kv.page_size) * v_row;
                    a = fmaf(ps[jj], gfb_to_f32(vrow[dim]), a);
                }
                acc[r] = a;
            }
        }
    }
    if (sink != nullptr) {
        // one more term in the denominator, exp(sink_h), with no value behind it
        const float sk = sink[h];
        const float m_fin = fmaxf(m_run, sk);
        const float corr = (m_run == -INFINITY) ? 0.f : expf(m_run - m_fin);
        l_run = l_run * corr + expf(sk - m_fin);
#pragma unroll
        for (int r = 0; r < MAX_DPT; r++) acc[r] *= corr;
    }
    float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    if (maps == 1) {
        T* orow = out + ((size_t)t * H + h) * dv;
#pragma unroll
        for (int r = 0; r < MAX_DPT; r++) {
            int dim = threadIdx.x + r * CHUNK;
            if (dim < dv) orow[dim] = gfb_from_f32<T>(acc[r] * inv);
        }
    } else if (map == 0) {
#pragma unroll
        for (int r = 0; r < MAX_DPT; r++) first[r] = acc[r] * inv;
    } else {
        // the difference of the two maps, normed over the head and scaled
        float ss = 0.f;
#pragma unroll
        for (int r = 0; r < MAX_DPT; r++) {
            first[r] -= lambda * (acc[r] * inv);
            if (threadIdx.x + r * CHUNK < dv) ss += first[r] * first[r];
        }
        __syncthreads();
        ss = gfb_block_sum(ss, scratch);
        const float f = out_scale / sqrtf(ss / (float)dv + diff_eps);
        T* orow = out + ((size_t)t * H + h) * dv;
#pragma unroll
        for (int r = 0; r < MAX_DPT; r++) {
            int dim = threadIdx.x + r * CHUNK;
            if (dim < dv) orow[dim] = gfb_from_f32<T>(first[r] * f);
        }
    }
  }
}

GFB_API int gfb_attention_generic(const void* q, void* out, int dt,
                                  void* k_pool, void* v_pool, const int* page_table, int max_pages, int page_size,
                                  int n_pages,
                                  const int* cu_seqlens, const int* tok_seq, const int* slots, const int* lengths,
                                  int n_seqs, int n_tokens, int H, int G, int d, int dv, float scale, int window,
                                  int chunk, const float* sink, int values_in_keys, const float* bias, int bias_len,
                                  const float* slopes, float softcap, int keep_first, int maps, float lambda, float diff_eps,
                                  float out_scale, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (maps != 1 && maps != 2) return gfb_fail("gfb_attention_generic: %d score maps per head (1 or 2)", maps);
    if (keep_first < 0) return gfb_fail("gfb_attention_generic: %d kept first positions", keep_first);
    if (keep_first > 0 && chunk > 0) return gfb_fail("gfb_attention_generic: kept first positions go with a window, not with a block mask");
    if (maps == 2 && (values_in_keys || sink != nullptr)) return gfb_fail("gfb_attention_generic: two maps take values of their own and no sink");
    if (dv <= 0) dv = d;
    if (dv > CHUNK * MAX_DPT) return gfb_fail("gfb_attention_generic: value head size %d exceeds %d", dv, CHUNK * MAX_DPT);
    if (G <= 0 || H % G) return gfb_fail("gfb_attention_generic: %d heads do not divide into %d groups", H, G);
    if (H > 65535) return gfb_fail("gfb_attention_generic: %d heads exceed the grid limit", H);
    if (bias != nullptr && bias_len < 1) return gfb_fail("gfb_attention_generic: a distance table of %d rows", bias_len);
    // values_in_keys: a value is the first dv dimensions of its key row (a latent shared by keys and values), so
    // the value pool is the key pool read with the keys' row stride
    if (values_in_keys && dv > d) return gfb_fail("gfb_attention_generic: values of %d dimensions inside keys of %d", dv, d);
    const int v_row = values_in_keys ? d : dv;
    GfbPagedKV kv{k_pool, values_in_keys ? k_pool : v_pool, page_table, max_pages, page_size, n_pages};
    GfbBatch b{cu_seqlens, tok_seq, slots, lengths, n_seqs, n_tokens};
    dim3 grid(n_tokens, H);
    size_t smem = (size_t)(d + CHUNK) * sizeof(float);
    cudaError_t e;
    if (dt == GFB_BF16)
        e = gfb_launch(attention_generic_kernel<__nv_bfloat16>, grid, dim3(CHUNK), smem, stream,
                       (const __nv_bfloat16*)q, (__nv_bfloat16*)out, kv, b, H, G, d, dv, v_row, scale, window, chunk, sink, bias, bias_len, slopes, softcap, keep_first, maps, lambda, diff_eps, out_scale, status);
    else if (dt == GFB_F32)
        e = gfb_launch(attention_generic_kernel<float>, grid, dim3(CHUNK), smem, stream,
                       (const float*)q, (float*)out, kv, b, H, G, d, dv, v_row, scale, window, chunk, sink, bias, bias_len, slopes, softcap, keep_first, maps, lambda, diff_eps, out_scale, status);
    else
        return gfb_fail("gfb_attention_generic: unknown type %d", dt);
    return gfb_check(e, "gfb_attention_generic");
}
