// Latent attention for bfloat16 on the tensor cores, for any step: whole prompts, continuations
// of a cached prefix and single decoded tokens.
//
// The cache holds ONE row of `d` values per token ([latent | rotated key part]); a row's first
// `dv` values are also its value.  Every query head brings a row of `d` values (its unrotated part
// already taken into the latent space), so all heads of all tokens read the same rows: the
// (token, head) pairs of a sequence are stacked, head fastest, into query rows, and a block owns
// 16 * RG consecutive ones (RG = 1, 2 or 4).  Row r belongs to token r / heads and sees keys up to that token's
// position.  p_j = exp(s_j) / (exp(sink_h) + sum_i exp(s_i)) with an optional learned sink per head.
// With `gate`, head h's output of token t is multiplied by sigmoid(gate[t, h]) while it is still
// float32 (a scalar per row, so it commutes with whatever matrix the values meet afterwards).
//
// Per tile of keys (half a page with 64 rows per block, a page with 32 or 16), with NW warps (8; 16
// when a block has 16 rows: such a block is bound by the latency of its short dependent steps):
//   A  scores: warp (row group, key group, value range) multiplies its 16 rows by its share of the keys
//      (mma.sync.m16n8k16, float32 accumulators) and leaves them in shared memory as float32; with 16
//      warps two share a group of 8 keys, each over half of the `d` values, and step B adds their
//      partial scores;
//   B  softmax: threads / rows threads per row: scale, mask, running maximum and sum in float32
//      (ex2.approx on scores pre-multiplied by log2 e); the weights go back to shared memory as TWO
//      bfloat16 terms (the rounded weight and what the rounding left over), so that they stay
//      float32 in effect through the second product;
//   C  output: warp w owns columns [w * 8 NT, (w + 1) * 8 NT) of the values for ALL rows of the
//      block and adds P V for both terms of P.
// Keys arrive through a two-stage cp.async ring; rows are padded by 16 bytes, which spreads the
// eight rows of every ldmatrix over distinct banks for any `d` that is a multiple of 16.
//
// With `n_splits` > 1 a block walks only its share of the key tiles and leaves an unnormalised
// partial output with its maximum and sum; bfi_attention_latent_bf16 then runs the merge.
#include "attention_tiles.cuh"

#define AL_PS(KT) ((KT) + 8)      // row stride of the weights' tiles, in bfloat16 (odd in 16-byte chunks)
#define AL_SS(KT) ((KT) + 1)      // row stride of the score tile, in float32
#define AL_LOG2E 1.4426950408889634f

__device__ __forceinline__ float al_gate(const bf16* gate, long gate_stride, long token, int h) {
    if (gate == nullptr) return 1.0f;
    const float x = __bfloat162float(gate[(size_t)token * gate_stride + h]);
    return 1.0f / (1.0f + expf(-x));          // expf(+large) = inf gives 0, expf(-large) = 0 gives 1
}

template <int RG, int NT, int AL_KEYS, int NW, int DS>
__global__ void __launch_bounds__(NW * 32, 1)
attention_latent_kernel(const bf16* __restrict__ q, long q_stride, bf16* __restrict__ out, long out_stride,
                        const bf16* __restrict__ pages, const int* __restrict__ block_table, int table_stride,
                        const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot,
                        const int* __restrict__ seq_start, int heads, int d, int dv, float scale_log2,
                        const float* __restrict__ sinks, const bf16* __restrict__ gate, long gate_stride, int n_splits,
                        float* __restrict__ part_o, float* __restrict__ part_ml) {
    constexpr int QR = 16 * RG;               // query rows of a block
    constexpr int THREADS = NW * 32;
    constexpr int KG = NW / (RG * DS);        // key groups in step A (DS warps share one, each with a range of the values)
    constexpr int KW = AL_KEYS / KG;          // keys of a warp in step A
    constexpr int KN = KW / 8;                // its score tiles of 8 keys
    constexpr int TPR = THREADS / QR;      // threads per row in step B
    constexpr int KPT = AL_KEYS / TPR;        // keys per thread in step B
    constexpr int PS = AL_PS(AL_KEYS), SS = AL_SS(AL_KEYS);
    pdl_trigger();
    pdl_wait();
    const int seq = blockIdx.z;
    const int slot = seq_slot[seq];
    if (slot < 0) return;
    const int t0 = cu_seqlens[seq];
    const int nt = cu_seqlens[seq + 1] - t0;
    const long n_rows = (long)nt * heads;
    // the last rows of a sequence walk the most keys: they start first
    const long row0 = (long)(gridDim.x - 1 - blockIdx.x) * QR;
    if (row0 >= n_rows) return;
    const int start = seq_start[seq];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int dp = d + 8;                     // padded row, in values

    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* qs = reinterpret_cast<bf16*>(smem_raw);                     // [QR][dp]
    bf16* ks[2] = {qs + QR * dp, qs + QR * dp + AL_KEYS * dp};        // [keys of a tile][dp] each
    bf16* ph = ks[1] + AL_KEYS * dp;                                  // [QR][PS] rounded weights
    bf16* pl = ph + QR * PS;                                       // [QR][PS] what the rounding left over
    float* ss = reinterpret_cast<float*>(pl + QR * PS);            // [DS][QR][SS] scores (DS partial sums each)
    float* corr_s = ss + DS * QR * SS;                             // [QR] factor for the running output
    float* m_s = corr_s + QR;                                         // [QR] final maximum
    float* l_s = m_s + QR;                                            // [QR] final sum
    __shared__ int tile_ok[2];

    // keys the block reads: 0 .. position of its last row's token
    const long last_row = min(row0 + QR, n_rows) - 1;
    const int hi_block = start + (int)(last_row / heads);
    const int n_tiles = hi_block / AL_KEYS + 1;
    const int per_split = (n_tiles + n_splits - 1) / n_splits;
    const int kt_beg = blockIdx.y * per_split;
    const int kt_end = min(kt_beg + per_split, n_tiles);             // exclusive

    const int chunks = d >> 3;
    const int* table = block_table + (size_t)slot * table_stride;
    auto issue = [&](int kt, int stage) {
        constexpr int PER_PAGE = BFI_PAGE_TOKENS / AL_KEYS;           // tiles of a page
        const int page = table[kt / PER_PAGE];
        if (threadIdx.x == 0) tile_ok[stage] = page >= 0;
        const bf16* src = pages + ((size_t)(page < 0 ? 0 : page) * BFI_PAGE_TOKENS + (size_t)(kt % PER_PAGE) * AL_KEYS) * d;
        const int key0 = kt * AL_KEYS;
        for (int row = warp; row < AL_KEYS; row += NW) {        // a warp per row, a lane per 16 bytes
            // rows that no query of the block sees may never have been written: zeros, so that a zero
            // weight times a stray NaN cannot reach the output
            const bool live = page >= 0 && key0 + row <= hi_block;
            for (int c = lane; c < chunks; c += 32) {
                bf16* dst = ks[stage] + row * dp + c * 8;
                if (live) cp_async16(dst, src + (size_t)row * d + c * 8);
                else *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        cp_async_commit();
    };

    // ---- the block's query rows -> shared memory (rows past the sequence are zero)
    for (int i = threadIdx.x; i < QR * chunks; i += THREADS) {
        const int row = i / chunks, c = i - row * chunks;
        bf16* dst = qs + row * dp + c * 8;
        const long r = row0 + row;
        if (r < n_rows) {
            const long tok = r / heads;
            const int h = (int)(r - tok * heads);
            cp_async16(dst, q + (size_t)(t0 + tok) * q_stride + (size_t)h * d + c * 8);
        } else {
            *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
        }
    }
    if (kt_beg < kt_end) issue(kt_beg, 0);        // the query copies ride in this first group
    else cp_async_commit();

    // step B's row of this thread
    const int brow = threadIdx.x / TPR, bsub = threadIdx.x % TPR;
    const long br = row0 + brow;
    const int bpos = br < n_rows ? start + (int)(br / heads) : -1;
    float m_run = -INFINITY, l_run = 0.0f;

    float o[RG][NT][4];
#pragma unroll
    for (int a = 0; a < RG; ++a)
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int c = 0; c < 4; ++c) o[a][n][c] = 0.0f;
    const int col0 = warp * 8 * NT;               // first value column of this warp in step C
    const int rg = warp % RG, kg = (warp / RG) % KG, ds = warp / (RG * KG);     // step A's row group, key group, value range

    for (int kt = kt_beg; kt < kt_end; ++kt) {
        const int stage = (kt - kt_beg) & 1;
        cp_async_wait<0>();
        __syncthreads();                          // tile kt is here; everyone has left step C of tile kt - 1
        if (kt + 1 < kt_end) issue(kt + 1, stage ^ 1);
        const bf16* ktile = ks[stage];

        // ---- A: scores of 16 rows x KW keys
        {
            float s[KN][4], s2[KN][4];            // even and odd steps: two chains of products, not one
#pragma unroll
            for (int j = 0; j < KN; ++j)
#pragma unroll
                for (int c = 0; c < 4; ++c) s[j][c] = s2[j][c] = 0.0f;
            const bf16* qrow = qs + (rg * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * dp + (lane >> 4) * 8;
            const bf16* krow = ktile + (kg * KW + (lane & 7)) * dp;
            // this warp's steps of 16 values: all of them, or one of DS ranges
            const int per_ds = ((d >> 4) + DS - 1) / DS;
            const int k_lo = ds * per_ds;
            const int ksteps = min(d >> 4, k_lo + per_ds);
            // two steps of 16 values per turn; the fragments of the next turn are asked for before this
            // turn's products, so the tensor cores do not wait for shared memory
            uint32_t a0[2][4], a1[2][4], b[2][KN][4];
            auto fetch = [&](int kk, int buf) {
                const bool two = kk + 1 < ksteps;
                ldmatrix_x4(a0[buf], qrow + kk * 16);
                ldmatrix_x4(a1[buf], qrow + (two ? kk + 1 : kk) * 16);
                // lanes 16..31 address the second step's chunks; without one they repeat the first's
                const int kc = 2 * kk + (two ? (lane >> 3) : ((lane >> 3) & 1));
#pragma unroll
                for (int j = 0; j < KN; ++j) ldmatrix_x4(b[buf][j], krow + j * 8 * dp + kc * 8);
            };
            if (k_lo < ksteps) fetch(k_lo, 0);
            int buf = 0;
            for (int kk = k_lo; kk < ksteps; kk += 2, buf ^= 1) {
                if (kk + 2 < ksteps) {
                    if (buf == 0) fetch(kk + 2, 1);
                    else fetch(kk + 2, 0);
                }
                const bool two = kk + 1 < ksteps;
#pragma unroll
                for (int j = 0; j < KN; ++j) {
                    if (buf == 0) {
                        mma16816(s[j], a0[0], b[0][j][0], b[0][j][1]);
                        if (two) mma16816(s2[j], a1[0], b[0][j][2], b[0][j][3]);
                    } else {
                        mma16816(s[j], a0[1], b[1][j][0], b[1][j][1]);
                        if (two) mma16816(s2[j], a1[1], b[1][j][2], b[1][j][3]);
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < KN; ++j) {
                float* dst = ss + (ds * QR + rg * 16 + g) * SS + kg * KW + j * 8 + 2 * t;
                dst[0] = s[j][0] + s2[j][0];
                dst[1] = s[j][1] + s2[j][1];
                dst[8 * SS] = s[j][2] + s2[j][2];
                dst[8 * SS + 1] = s[j][3] + s2[j][3];
            }
        }
        __syncthreads();

        // ---- B: softmax of this thread's row over its KPT keys
        bool moved;
        {
            const bool ok = tile_ok[stage] != 0;
            float v[KPT];
            float mx = -INFINITY;
#pragma unroll
            for (int i = 0; i < KPT; ++i) {
                const int key = kt * AL_KEYS + bsub * KPT + i;
                float x = ss[brow * SS + bsub * KPT + i];
                if (DS == 2) x += ss[(QR + brow) * SS + bsub * KPT + i];
                x *= scale_log2;
                if (!ok || key > bpos) x = -INFINITY;
                v[i] = x;
                mx = fmaxf(mx, x);
            }
#pragma unroll
            for (int w = 1; w < TPR; w <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, w));
            const float m_new = fmaxf(m_run, mx);
            const float corr = (m_run == -INFINITY) ? 0.0f : fast_exp2(m_run - m_new);
            float sum = 0.0f;
            uint32_t hi[KPT / 2], lo[KPT / 2];
#pragma unroll
            for (int i = 0; i < KPT; i += 2) {
                const float p0 = (v[i] == -INFINITY) ? 0.0f : fast_exp2(v[i] - m_new);
                const float p1 = (v[i + 1] == -INFINITY) ? 0.0f : fast_exp2(v[i + 1] - m_new);
                sum += p0 + p1;
                hi[i / 2] = pack_bf16(p0, p1);
                lo[i / 2] = pack_bf16(p0 - bf16_lo(hi[i / 2]), p1 - bf16_hi(hi[i / 2]));
            }
#pragma unroll
            for (int w = 1; w < TPR; w <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, w);
            l_run = l_run * corr + sum;
            m_run = m_new;
            uint32_t* dh = reinterpret_cast<uint32_t*>(ph + brow * PS + bsub * KPT);
            uint32_t* dl = reinterpret_cast<uint32_t*>(pl + brow * PS + bsub * KPT);
#pragma unroll
            for (int i = 0; i < KPT / 2; ++i) {
                dh[i] = hi[i];
                dl[i] = lo[i];
            }
            if (bsub == 0) corr_s[brow] = corr;
            moved = corr != 1.0f && m_new != -INFINITY;      // a row that has seen no key has nothing to rescale
        }
        const bool rescale = __syncthreads_or(moved);     // once the maxima have settled nothing is rescaled

        // ---- C: output += P V over this warp's columns, all rows
        if (col0 < dv) {
            if (rescale)
#pragma unroll
            for (int a = 0; a < RG; ++a) {
                const float c0 = corr_s[a * 16 + g], c1 = corr_s[a * 16 + g + 8];
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    o[a][n][0] *= c0;
                    o[a][n][1] *= c0;
                    o[a][n][2] *= c1;
                    o[a][n][3] *= c1;
                }
            }
#pragma unroll
            for (int k16 = 0; k16 < AL_KEYS / 16; ++k16) {
                uint32_t ah[RG][4], al[RG][4];
#pragma unroll
                for (int a = 0; a < RG; ++a) {
                    const int off = (a * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * PS + k16 * 16 + (lane >> 4) * 8;
                    ldmatrix_x4(ah[a], ph + off);
                    ldmatrix_x4(al[a], pl + off);
                }
                const bf16* vrow = ktile + (k16 * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * dp + col0 + (lane >> 4) * 8;
#pragma unroll
                for (int n = 0; n < NT; n += 2) {
                    if (col0 + n * 8 >= dv) break;            // the same for the whole warp
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, vrow + n * 8);
#pragma unroll
                    for (int a = 0; a < RG; ++a) {
                        mma16816(o[a][n], ah[a], b[0], b[1]);
                        mma16816(o[a][n + 1], ah[a], b[2], b[3]);
                    }
#pragma unroll
                    for (int a = 0; a < RG; ++a) {
                        mma16816(o[a][n], al[a], b[0], b[1]);
                        mma16816(o[a][n + 1], al[a], b[2], b[3]);
                    }
                }
            }
        }
    }
    cp_async_wait<0>();

    // ---- the rows' maxima and sums to the threads that hold the output
    __syncthreads();
    if (bsub == 0) {
        m_s[brow] = m_run;
        l_s[brow] = l_run;
    }
    __syncthreads();
    if (col0 >= dv) return;
#pragma unroll
    for (int a = 0; a < RG; ++a)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int row = a * 16 + g + half * 8;
            const long r = row0 + row;
            if (r >= n_rows) continue;
            const long tok = r / heads;
            const int h = (int)(r - tok * heads);
            const float m = m_s[row], l = l_s[row];
            if (n_splits > 1) {
                const size_t pr = ((size_t)t0 * heads + r) * n_splits + blockIdx.y;
                float* po = part_o + pr * dv;
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    const int col = col0 + n * 8 + 2 * t;
                    if (col < dv) *reinterpret_cast<float2*>(po + col) = make_float2(o[a][n][half * 2], o[a][n][half * 2 + 1]);
                }
                if (warp == 0 && t == 0) {
                    part_ml[pr * 2] = m;
                    part_ml[pr * 2 + 1] = l;
                }
            } else {
                float l_all = l;
                if (sinks != nullptr && m > -INFINITY) l_all += fast_exp2(sinks[h] * AL_LOG2E - m);
                const float inv = l_all > 0.0f ? al_gate(gate, gate_stride, t0 + tok, h) / l_all : 0.0f;
                bf16* orow = out + (size_t)(t0 + tok) * out_stride + (size_t)h * dv;
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    const int col = col0 + n * 8 + 2 * t;
                    if (col < dv)
                        *reinterpret_cast<__nv_bfloat162*>(orow + col) =
                            __floats2bfloat162_rn(o[a][n][half * 2] * inv, o[a][n][half * 2 + 1] * inv);
                }
            }
        }
}

// One block per query row: the partial outputs of the row's key ranges, each with its maximum and
// sum, become the row's output; the sink's term joins the denominator here.
__global__ void __launch_bounds__(128)
attention_latent_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, bf16* __restrict__ out,
                              long out_stride, const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot,
                              int heads, int dv, int n_splits, const float* __restrict__ sinks,
                              const bf16* __restrict__ gate, long gate_stride) {
    pdl_trigger();
    pdl_wait();
    const int seq = blockIdx.z;
    if (seq_slot[seq] < 0) return;
    const int t0 = cu_seqlens[seq];
    const int nt = cu_seqlens[seq + 1] - t0;
    const long r = blockIdx.x;
    if (r >= (long)nt * heads) return;
    const long tok = r / heads;
    const int h = (int)(r - tok * heads);
    const size_t pr = ((size_t)t0 * heads + r) * n_splits;
    float m = -INFINITY;
    for (int z = 0; z < n_splits; ++z) m = fmaxf(m, part_ml[(pr + z) * 2]);
    float l = 0.0f;
    for (int z = 0; z < n_splits; ++z) {
        const float mz = part_ml[(pr + z) * 2];
        if (mz > -INFINITY) l += part_ml[(pr + z) * 2 + 1] * fast_exp2(mz - m);
    }
    if (sinks != nullptr && m > -INFINITY) l += fast_exp2(sinks[h] * AL_LOG2E - m);
    const float inv = l > 0.0f ? al_gate(gate, gate_stride, t0 + tok, h) / l : 0.0f;
    bf16* orow = out + (size_t)(t0 + tok) * out_stride + (size_t)h * dv;
    for (int c = threadIdx.x; c < dv; c += blockDim.x) {
        float acc = 0.0f;
        for (int z = 0; z < n_splits; ++z) {
            const float mz = part_ml[(pr + z) * 2];
            if (mz > -INFINITY) acc = fmaf(part_o[(pr + z) * dv + c], fast_exp2(mz - m), acc);
        }
        orow[c] = __float2bfloat16(acc * inv);
    }
}

static size_t latent_smem(int rows, int keys, int d, int ds = 1) {
    return (size_t)(rows + 2 * keys) * (d + 8) * sizeof(bf16) + (size_t)2 * rows * AL_PS(keys) * sizeof(bf16) +
           (size_t)ds * rows * AL_SS(keys) * sizeof(float) + (size_t)3 * rows * sizeof(float);
}

template <int RG, int NT, int KT, int NW, int DS>
static int launch_latent(const void* q, long q_stride, void* out, long out_stride, const void* pages, const int* block_table,
                         int table_stride, const int* cu_seqlens, const int* seq_slot, const int* seq_start, int n_seqs,
                         int max_tokens, int heads, int d, int dv, float scale, const float* sinks, const bf16* gate,
                         long gate_stride, int n_splits, float* part_o, float* part_ml, cudaStream_t stream) {
    constexpr int QR = 16 * RG;
    static_assert((DS == 1 || DS == 2) && NW % (RG * DS) == 0 && (KT * RG * DS) % (8 * NW) == 0 && (NW * 32) % QR == 0 &&
                  (KT * QR) % (64 * NW) == 0, "a warp takes whole groups of 8 keys, a thread an even number of keys of its row");
    const size_t smem = latent_smem(QR, KT, d, DS);
    auto kernel = attention_latent_kernel<RG, NT, KT, NW, DS>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return bfi_fail("attention_latent: cannot reserve %zu bytes of shared memory: %s", smem,
                                              cudaGetErrorString(e));
    }
    const long rows = (long)max_tokens * heads;
    dim3 grid((unsigned)((rows + QR - 1) / QR), n_splits, n_seqs);
    bfi_launch(kernel, grid, dim3(NW * 32), smem, stream, (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)pages,
               block_table, table_stride, cu_seqlens, seq_slot, seq_start, heads, d, dv, scale * AL_LOG2E, sinks, gate, gate_stride,
               n_splits, part_o, part_ml);
    if (bfi_check_launch("attention_latent")) return 1;
    if (n_splits > 1) {
        bfi_launch(attention_latent_merge_kernel, dim3((unsigned)rows, 1, n_seqs), dim3(128), 0, stream, (const float*)part_o,
                   (const float*)part_ml, (bf16*)out, out_stride, cu_seqlens, seq_slot, heads, dv, n_splits, sinks, gate, gate_stride);
        return bfi_check_launch("attention_latent_merge");
    }
    return 0;
}

// Returns 0 on success, 1 on error, 2 when the shape is not taken (nothing launched).
// `q` rows are [heads][d] per token, `out` rows [heads][dv]; `pages` is the cache ([pages][64 tokens][d]);
// `sinks`: float32, one per head, or null.  `gate`: bfloat16 logits, [tokens][heads] with `gate_stride`
// values between tokens, or null.  `n_splits` > 1 needs `part_o` (tokens * heads * n_splits * dv
// floats) and `part_ml` (tokens * heads * n_splits * 2 floats).
extern "C" int bfi_attention_latent_bf16(const void* q, long q_stride, void* out, long out_stride, const void* pages,
                                         const int* block_table, int table_stride, const int* cu_seqlens,
                                         const int* seq_slot, const int* seq_start, int n_seqs, int max_tokens, int heads,
                                         int d, int dv, float scale, const float* sinks, const void* gate,
                                         long gate_stride, int n_splits, float* part_o, float* part_ml,
                                         cudaStream_t stream) {
    BFI_REQUIRE(heads > 0 && d > 0 && dv > 0 && dv <= d, "attention_latent: bad sizes heads=%d d=%d dv=%d", heads, d, dv);
    BFI_REQUIRE(n_splits >= 1 && (n_splits == 1 || (part_o != nullptr && part_ml != nullptr)),
                "attention_latent: %d key ranges need their scratch", n_splits);
    if (n_seqs <= 0 || max_tokens <= 0) return 0;
    if (d % 16 != 0 || dv % 16 != 0 || dv > 512 || d > 768) return 2;
    if (q_stride % 8 != 0 || out_stride % 2 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)out & 3) || ((uintptr_t)pages & 15) ||
        n_seqs > 65535 || n_splits > 65535)
        return 2;
    if (latent_smem(64, 32, d) > 227 * 1024) return 2;
#define BFI_AL_CASE(RG, NT, KT, NW, DS)                                                                                      \
    return launch_latent<RG, NT, KT, NW, DS>(q, q_stride, out, out_stride, pages, block_table, table_stride, cu_seqlens, seq_slot, \
                                 seq_start, n_seqs, max_tokens, heads, d, dv, scale, sinks, (const bf16*)gate, gate_stride, n_splits, part_o,   \
                                 part_ml, stream)
    // few rows: blocks of 16 or 32 rows that take a whole page of keys per turn, where that fits.  A
    // block of 16 rows (single tokens of up to 16 heads) is bound by the latency of its short dependent
    // steps, so it has 16 warps: two share a group of 8 keys, each over half of the row's values (with
    // 32 rows the same made no difference: 186 against 181 us at 64 sequences of 4,096 tokens)
    const long rows = (long)max_tokens * heads;
    const bool few = rows <= 32 && latent_smem(32, 64, d) <= 227 * 1024;
    if (rows <= 16 && latent_smem(16, 64, d, 2) <= 227 * 1024) {
        if (dv <= 256) BFI_AL_CASE(1, 2, 64, 16, 2);
        BFI_AL_CASE(1, 4, 64, 16, 2);
    }
    if (few) {
        if (dv <= 128) BFI_AL_CASE(2, 2, 64, 8, 1);
        if (dv <= 256) BFI_AL_CASE(2, 4, 64, 8, 1);
        BFI_AL_CASE(2, 8, 64, 8, 1);
    }
    if (dv <= 128) BFI_AL_CASE(4, 2, 32, 8, 1);
    if (dv <= 256) BFI_AL_CASE(4, 4, 32, 8, 1);
    BFI_AL_CASE(4, 8, 32, 8, 1);
#undef BFI_AL_CASE
}
