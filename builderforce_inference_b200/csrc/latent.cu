// Latent attention: keys and values of all heads are made from one small vector per token (the
// latent c, `rank` values, RMS-normed) and one rotated key part (`rd` values) that all heads share.
// Only those rank + rd values are cached per token; the cache row is [c | rotated part], ONE
// key/value "head" whose values are the first `rank` values of its keys.
//
// With per-head matrices W_uk [heads * d, rank] (unrotated keys k_h = W_uk_h c) and W_uv
// [heads * dv, rank] (values v_h = W_uv_h c), the score of query head h against a cached token is
//     (q_h^n . W_uk_h c + q_h^r . k^r) * scale = ((W_uk_h^T q_h^n) . c + q_h^r . k^r) * scale
// and its output  sum_j p_j W_uv_h c_j = W_uv_h (sum_j p_j c_j).  So the attention itself runs in
// the latent space: every query head becomes [W_uk_h^T q_h^n | rot(q_h^r)] (rank + rd values), all
// heads read the same cached rows, the weighted sum of the c_j comes back (rank values per head),
// and W_uv_h takes it to the head's dv values.  Nothing is expanded per cached token.
//
// Kernels (float32 arithmetic; storage float32 or bfloat16):
//   bfi_latent_prepare  per token: the query heads' rotated parts turned by the token's angles and
//                       put behind the absorbed part's place in the query buffer; the latent normed,
//                       the shared key part turned, both written to the token's cache row.
//   bfi_latent_absorb   qa[t, h, 0..rank) = W_uk_h^T q[t, h, 0..d)
//   bfi_latent_expand   o[t, h, :] = (W_uv_h lat[t, h, :]) * sigmoid(gate[t, h])   (gate optional)
//
// A projections row is [heads * (d + rd) queries, head by head as d unrotated then rd rotated |
// `gates` gate logits | rank + rd of the down projection (absent in a layer that borrows another
// layer's cache)].  The rotation pairs value i with value i + rot_dim/2 of the rotated part's first
// rot_dim values; the rest pass.
#include "common.cuh"

#define LAT_THREADS 256

template <typename T>
__global__ void __launch_bounds__(LAT_THREADS)
latent_prepare_kernel(const T* __restrict__ proj, long proj_stride, T* __restrict__ qa, long qa_stride, int n_heads, int d,
                      int rd, int rank, int kv_off, const void* __restrict__ norm_w, int norm_dtype, float eps,
                      const float2* __restrict__ rope, int rot_dim, int table_positions, const int* __restrict__ token_pos,
                      const int* __restrict__ token_slot, T* __restrict__ k_pages, const int* __restrict__ block_table,
                      int table_stride, int write_cache, int* __restrict__ status) {
    pdl_trigger();
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const int slot = token_slot[t];
    if (slot < 0) return;                         // padding row
    const int pos = token_pos[t];
    const bool bad_pos = rot_dim > 0 && (pos < 0 || pos >= table_positions);
    int page = -1;
    if (write_cache) page = block_table[(size_t)slot * table_stride + pos / BFI_PAGE_TOKENS];
    pdl_wait();
    if (bad_pos) {
        if (threadIdx.x == 0 && status) atomicOr(status, BFI_STATUS_BAD_POSITION);
    }
    const T* row = proj + (size_t)t * proj_stride;
    const int half = rot_dim >> 1;
    const float2* ang = (rot_dim > 0 && !bad_pos) ? rope + (size_t)pos * half : nullptr;
    const int dq = d + rd;

    // ---- the query heads' rotated parts
    T* qrow = qa + (size_t)t * qa_stride;
    for (int i = threadIdx.x; i < n_heads * rd; i += LAT_THREADS) {
        const int h = i / rd, e = i - h * rd;
        const T* src = row + (size_t)h * dq + d;
        float v = to_f32(src[e]);
        if (ang != nullptr && e < rot_dim) {
            const int f = e < half ? e : e - half;
            const float2 cs = ang[f];
            const float other = to_f32(src[e < half ? e + half : e - half]);
            v = e < half ? v * cs.x - other * cs.y : v * cs.x + other * cs.y;
        }
        qrow[(size_t)h * (rank + rd) + rank + e] = from_f32<T>(v);
    }
    if (!write_cache) return;
    if (page < 0) {
        if (threadIdx.x == 0 && status) atomicOr(status, BFI_STATUS_NO_PAGE);
        return;
    }
    // ---- the latent, normed, and the shared key part, turned, into the token's cache row
    const T* kv = row + kv_off;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < rank; j += LAT_THREADS) {
        const float v = to_f32(kv[j]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)rank + eps);
    T* dst = k_pages + ((size_t)page * BFI_PAGE_TOKENS + (pos % BFI_PAGE_TOKENS)) * (rank + rd);
    for (int j = threadIdx.x; j < rank + rd; j += LAT_THREADS) {
        float v = to_f32(kv[j]);
        if (j < rank) {
            v = v * inv * load_as_f32(norm_w, norm_dtype, j);
        } else if (ang != nullptr && j - rank < rot_dim) {
            const int e = j - rank;
            const int f = e < half ? e : e - half;
            const float2 cs = ang[f];
            const float other = to_f32(kv[rank + (e < half ? e + half : e - half)]);
            v = e < half ? v * cs.x - other * cs.y : v * cs.x + other * cs.y;
        }
        dst[j] = from_f32<T>(v);
    }
}

extern "C" int bfi_latent_prepare(const void* proj, int dtype, long proj_stride, void* qa, long qa_stride, int n_tokens,
                                  int n_heads, int d, int rd, int rank, int kv_off, const void* norm_w, int norm_dtype,
                                  float eps, const float* rope, int rot_dim, int table_positions, const int* token_pos,
                                  const int* token_slot, void* k_pages, const int* block_table, int table_stride,
                                  int write_cache, int* status, cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(dtype) && dtype_ok(norm_dtype), "latent_prepare: unknown dtype code");
    BFI_REQUIRE(n_heads > 0 && d >= 0 && rd >= 0 && rank > 0, "latent_prepare: bad sizes heads=%d d=%d rd=%d rank=%d", n_heads,
                d, rd, rank);
    BFI_REQUIRE(rot_dim >= 0 && rot_dim % 2 == 0 && rot_dim <= rd, "latent_prepare: %d rotated values of %d", rot_dim, rd);
    BFI_REQUIRE(rot_dim == 0 || rope != nullptr, "latent_prepare: a rotation needs its table");
    BFI_REQUIRE(qa_stride >= (long)n_heads * (rank + rd), "latent_prepare: the query buffer's rows are too short");
    if (write_cache)
        BFI_REQUIRE(k_pages && block_table && norm_w && proj_stride >= (long)kv_off + rank + rd,
                    "latent_prepare: writing the cache needs pages, a page table, the norm's weight and the down projection");
    if (n_tokens <= 0) return 0;
    if (dtype == BFI_F32)
        bfi_launch(latent_prepare_kernel<float>, dim3(n_tokens), dim3(LAT_THREADS), 0, stream, (const float*)proj, proj_stride,
                   (float*)qa, qa_stride, n_heads, d, rd, rank, kv_off, norm_w, norm_dtype, eps, (const float2*)rope, rot_dim,
                   table_positions, token_pos, token_slot, (float*)k_pages, block_table, table_stride, write_cache, status);
    else
        bfi_launch(latent_prepare_kernel<bf16>, dim3(n_tokens), dim3(LAT_THREADS), 0, stream, (const bf16*)proj, proj_stride,
                   (bf16*)qa, qa_stride, n_heads, d, rd, rank, kv_off, norm_w, norm_dtype, eps, (const float2*)rope, rot_dim,
                   table_positions, token_pos, token_slot, (bf16*)k_pages, block_table, table_stride, write_cache, status);
    return bfi_check_launch("latent_prepare");
}

// ------------------------------------------------------------------------------------------
// qa[t, h, j] = sum_e W_uk[h * d + e, j] * q[t, h, e]       j < rank
// grid (token tiles, heads, column groups); a block stages LAT_TOK tokens' unrotated query values of
// its head as float32 and walks its LAT_COLS columns of W_uk_h once for all of them: a thread owns
// one column, so a row of W_uk_h is read by consecutive threads.  Few tokens still make heads *
// rank / LAT_COLS blocks.
// ------------------------------------------------------------------------------------------
#define LAT_TOK 8
#define LAT_COLS 64

template <typename T, typename TW>
__global__ void __launch_bounds__(LAT_COLS)
latent_absorb_kernel(const T* __restrict__ proj, long proj_stride, const TW* __restrict__ w_uk, T* __restrict__ qa,
                     long qa_stride, const int* __restrict__ token_slot, int n_tokens, int d, int rd, int rank) {
    pdl_trigger();
    extern __shared__ float qs[];                 // [LAT_TOK][d]
    const int h = blockIdx.y;
    const int t0 = blockIdx.x * LAT_TOK;
    pdl_wait();
    for (int i = threadIdx.x; i < LAT_TOK * d; i += LAT_COLS) {
        const int tt = i / d, e = i - tt * d;
        const int t = t0 + tt;
        qs[i] = (t < n_tokens && token_slot[t] >= 0) ? to_f32(proj[(size_t)t * proj_stride + (size_t)h * (d + rd) + e]) : 0.0f;
    }
    __syncthreads();
    const TW* w = w_uk + (size_t)h * d * rank;
    const int j = blockIdx.z * LAT_COLS + threadIdx.x;
    if (j < rank) {
        float acc[LAT_TOK];
#pragma unroll
        for (int tt = 0; tt < LAT_TOK; ++tt) acc[tt] = 0.0f;
        for (int e = 0; e < d; ++e) {
            const float wv = to_f32(w[(size_t)e * rank + j]);
#pragma unroll
            for (int tt = 0; tt < LAT_TOK; ++tt) acc[tt] = fmaf(wv, qs[tt * d + e], acc[tt]);
        }
#pragma unroll
        for (int tt = 0; tt < LAT_TOK; ++tt) {
            const int t = t0 + tt;
            if (t < n_tokens && token_slot[t] >= 0) qa[(size_t)t * qa_stride + (size_t)h * (rank + rd) + j] = from_f32<T>(acc[tt]);
        }
    }
}

extern "C" int bfi_latent_absorb(const void* proj, int dtype, long proj_stride, const void* w_uk, int w_dtype, void* qa,
                                 long qa_stride, const int* token_slot, int n_tokens, int n_heads, int d, int rd, int rank,
                                 cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(dtype) && dtype_ok(w_dtype), "latent_absorb: unknown dtype code");
    BFI_REQUIRE(n_heads > 0 && n_heads <= 65535 && d > 0 && rd >= 0 && rank > 0, "latent_absorb: bad sizes");
    BFI_REQUIRE(dtype == w_dtype || w_dtype == BFI_F32, "latent_absorb: weights of the activations' type or float32");
    BFI_REQUIRE((size_t)LAT_TOK * d * 4 <= 48 * 1024, "latent_absorb: %d unrotated values per head are too many", d);
    if (n_tokens <= 0) return 0;
    const dim3 grid((n_tokens + LAT_TOK - 1) / LAT_TOK, n_heads, (rank + LAT_COLS - 1) / LAT_COLS);
    BFI_REQUIRE(grid.z <= 65535, "latent_absorb: a latent of %d values is too large", rank);
    const size_t smem = (size_t)LAT_TOK * d * sizeof(float);
    if (dtype == BFI_F32)
        bfi_launch(latent_absorb_kernel<float, float>, grid, dim3(LAT_COLS), smem, stream, (const float*)proj, proj_stride,
                   (const float*)w_uk, (float*)qa, qa_stride, token_slot, n_tokens, d, rd, rank);
    else if (w_dtype == BFI_F32)
        bfi_launch(latent_absorb_kernel<bf16, float>, grid, dim3(LAT_COLS), smem, stream, (const bf16*)proj, proj_stride,
                   (const float*)w_uk, (bf16*)qa, qa_stride, token_slot, n_tokens, d, rd, rank);
    else
        bfi_launch(latent_absorb_kernel<bf16, bf16>, grid, dim3(LAT_COLS), smem, stream, (const bf16*)proj, proj_stride,
                   (const bf16*)w_uk, (bf16*)qa, qa_stride, token_slot, n_tokens, d, rd, rank);
    return bfi_check_launch("latent_absorb");
}

// ------------------------------------------------------------------------------------------
// o[t, h * dv + i] = (sum_j W_uv[h * dv + i, j] * lat[t, h * rank + j]) * sigmoid(gate[t, h])
// grid (token tiles, heads, groups of 8 outputs); a block stages LAT_TOK tokens' latent outputs of
// its head as float32; a warp owns ONE output row i of the head and walks W_uv's row once for all
// staged tokens.  Few tokens still make heads * dv / 8 blocks.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float lat_sigmoid(float x) {
    if (x >= 0.0f) return 1.0f / (1.0f + expf(-x));
    const float z = expf(x);
    return z / (1.0f + z);
}

template <typename T, typename TW>
__global__ void __launch_bounds__(LAT_THREADS)
latent_expand_kernel(const T* __restrict__ lat, long lat_stride, const TW* __restrict__ w_uv, const T* __restrict__ gate,
                     long gate_stride, T* __restrict__ out, long out_stride, const int* __restrict__ token_slot, int n_tokens,
                     int dv, int rank, int gate_values) {
    pdl_trigger();
    extern __shared__ float ls[];                 // [LAT_TOK][rank] then [LAT_TOK] gates
    float* gs = ls + LAT_TOK * rank;
    const int h = blockIdx.y;
    const int t0 = blockIdx.x * LAT_TOK;
    pdl_wait();
    for (int i = threadIdx.x; i < LAT_TOK * rank; i += LAT_THREADS) {
        const int tt = i / rank, j = i - tt * rank;
        const int t = t0 + tt;
        ls[i] = (t < n_tokens && token_slot[t] >= 0) ? to_f32(lat[(size_t)t * lat_stride + (size_t)h * rank + j]) : 0.0f;
    }
    if (threadIdx.x < LAT_TOK) {
        const int t = t0 + threadIdx.x;
        float g = 1.0f;
        if (gate != nullptr && !gate_values && t < n_tokens && token_slot[t] >= 0)
            g = lat_sigmoid(to_f32(gate[(size_t)t * gate_stride + h]));
        gs[threadIdx.x] = g;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int i = blockIdx.z * (LAT_THREADS / 32) + warp;
    if (i < dv) {
        const TW* w = w_uv + ((size_t)h * dv + i) * rank;
        float acc[LAT_TOK];
#pragma unroll
        for (int tt = 0; tt < LAT_TOK; ++tt) acc[tt] = 0.0f;
        for (int j = lane; j < rank; j += 32) {
            const float wv = to_f32(w[j]);
#pragma unroll
            for (int tt = 0; tt < LAT_TOK; ++tt) acc[tt] = fmaf(wv, ls[tt * rank + j], acc[tt]);
        }
#pragma unroll
        for (int tt = 0; tt < LAT_TOK; ++tt) acc[tt] = warp_sum(acc[tt]);
        if (lane == 0) {
#pragma unroll
            for (int tt = 0; tt < LAT_TOK; ++tt) {
                const int t = t0 + tt;
                if (t < n_tokens && token_slot[t] >= 0) {
                    float g = gs[tt];
                    if (gate != nullptr && gate_values)      // a gate per value, laid out like the output
                        g = lat_sigmoid(to_f32(gate[(size_t)t * gate_stride + (size_t)h * dv + i]));
                    out[(size_t)t * out_stride + (size_t)h * dv + i] = from_f32<T>(acc[tt] * g);
                }
            }
        }
    }
}

extern "C" int bfi_latent_expand(const void* lat, int dtype, long lat_stride, const void* w_uv, int w_dtype, const void* gate,
                                 long gate_stride, void* out, long out_stride, const int* token_slot, int n_tokens, int n_heads,
                                 int dv, int rank, int gate_values, cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(dtype) && dtype_ok(w_dtype), "latent_expand: unknown dtype code");
    BFI_REQUIRE(n_heads > 0 && n_heads <= 65535 && dv > 0 && rank > 0, "latent_expand: bad sizes");
    BFI_REQUIRE(dtype == w_dtype || w_dtype == BFI_F32, "latent_expand: weights of the activations' type or float32");
    BFI_REQUIRE(lat_stride >= (long)n_heads * rank && out_stride >= (long)n_heads * dv, "latent_expand: rows shorter than the heads");
    const size_t smem = (size_t)(LAT_TOK * rank + LAT_TOK) * sizeof(float);
    BFI_REQUIRE(smem <= 48 * 1024, "latent_expand: a latent of %d values is too large", rank);
    if (n_tokens <= 0) return 0;
    const dim3 grid((n_tokens + LAT_TOK - 1) / LAT_TOK, n_heads, (dv + LAT_THREADS / 32 - 1) / (LAT_THREADS / 32));
    BFI_REQUIRE(grid.z <= 65535, "latent_expand: heads of %d values are too large", dv);
    if (dtype == BFI_F32)
        bfi_launch(latent_expand_kernel<float, float>, grid, dim3(LAT_THREADS), smem, stream, (const float*)lat, lat_stride,
                   (const float*)w_uv, (const float*)gate, gate_stride, (float*)out, out_stride, token_slot, n_tokens, dv, rank, gate_values);
    else if (w_dtype == BFI_F32)
        bfi_launch(latent_expand_kernel<bf16, float>, grid, dim3(LAT_THREADS), smem, stream, (const bf16*)lat, lat_stride,
                   (const float*)w_uv, (const bf16*)gate, gate_stride, (bf16*)out, out_stride, token_slot, n_tokens, dv, rank, gate_values);
    else
        bfi_launch(latent_expand_kernel<bf16, bf16>, grid, dim3(LAT_THREADS), smem, stream, (const bf16*)lat, lat_stride,
                   (const bf16*)w_uv, (const bf16*)gate, gate_stride, (bf16*)out, out_stride, token_slot, n_tokens, dv, rank, gate_values);
    return bfi_check_launch("latent_expand");
}

// ------------------------------------------------------------------------------------------
// A hashed bigram embedding, added to the residual stream: x[t] += table[row(t)] with
//     row = (previous token * mul_prev + token * mul_cur) mod buckets,
// and row `buckets` (the table's last) for a sequence's first token.  The previous token of a
// step's first token of a sequence is what the sequence's state holds (`last_token[slot]`); of the
// others it is the row before.  bfi_keep_last_tokens then moves the state on to the step's last
// token of every sequence (a launch of its own: it overwrites what the first kernel reads).
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void bigram_add_kernel(const T* __restrict__ table, const int* __restrict__ ids, const int* __restrict__ token_pos,
                                  const int* __restrict__ token_slot, const int* __restrict__ last_token,
                                  float* __restrict__ x, int width, int buckets, long long mul_prev, long long mul_cur,
                                  int vocab, int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int slot = token_slot[t];
    if (slot < 0) return;
    const int id = ids[t];
    if (id < 0 || id >= vocab) return;            // the embedding has recorded it
    int r = buckets;
    if (token_pos[t] > 0) {
        const int prev = (t > 0 && token_slot[t - 1] == slot) ? ids[t - 1] : last_token[slot];
        if (prev < 0 || prev >= vocab) {
            if (threadIdx.x == 0 && status) atomicOr(status, BFI_STATUS_BAD_TOKEN);
            return;
        }
        r = (int)(((long long)prev * mul_prev + (long long)id * mul_cur) % (long long)buckets);
    }
    const T* row = table + (size_t)r * width;
    float* o = x + (size_t)t * width;
    for (int j = threadIdx.x; j < width; j += blockDim.x) o[j] += to_f32(row[j]);
}

extern "C" int bfi_bigram_add(const void* table, int table_dtype, const int* ids, const int* token_pos, const int* token_slot,
                              const int* last_token, float* x, int n_tokens, int width, int buckets, long mul_prev,
                              long mul_cur, int vocab, int* status, cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(table_dtype), "bigram_add: unknown table dtype code %d", table_dtype);
    BFI_REQUIRE(width > 0 && buckets > 0 && mul_prev >= 0 && mul_cur >= 0 && vocab > 0, "bigram_add: bad sizes or multipliers");
    if (n_tokens <= 0) return 0;
    const int threads = width >= 1024 ? 256 : 128;
    if (table_dtype == BFI_F32)
        bfi_launch(bigram_add_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, (const float*)table, ids, token_pos,
                   token_slot, last_token, x, width, buckets, (long long)mul_prev, (long long)mul_cur, vocab, status);
    else
        bfi_launch(bigram_add_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, stream, (const bf16*)table, ids, token_pos,
                   token_slot, last_token, x, width, buckets, (long long)mul_prev, (long long)mul_cur, vocab, status);
    return bfi_check_launch("bigram_add");
}

__global__ void keep_last_tokens_kernel(const int* __restrict__ ids, const int* __restrict__ cu_seqlens,
                                        const int* __restrict__ seq_slot, int* __restrict__ last_token, int n_seqs) {
    pdl_trigger();
    pdl_wait();
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= n_seqs) return;
    const int slot = seq_slot[s];
    const int a = cu_seqlens[s], b = cu_seqlens[s + 1];
    if (slot >= 0 && b > a) last_token[slot] = ids[b - 1];
}

extern "C" int bfi_keep_last_tokens(const int* ids, const int* cu_seqlens, const int* seq_slot, int* last_token, int n_seqs,
                                    cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    bfi_launch(keep_last_tokens_kernel, dim3((n_seqs + 127) / 128), dim3(128), 0, stream, ids, cu_seqlens, seq_slot, last_token,
               n_seqs);
    return bfi_check_launch("keep_last_tokens");
}

BFI_TRACE_EXPORT(latent)
