// Work that goes channel by channel over the step's tokens.
//
// bfi_gated_scan: a recurrence with one state value per channel whose gates read the current token
//     only (minGRU).  With z_t = sigmoid(zr_t + b_z) and u_t = ur_t + b_u, where zr and ur are two
//     column ranges of the projections,
//         S_t = (1 - z_t) S_(t-1) + z_t cand(u_t)          y_t = S_t * act(g_t)
//     cand is the identity (0) or the positive map  u + 1/2 for u >= 0, sigmoid(u) for u < 0  (1);
//     act is silu of a third column range, or absent.  S lives in float32 per slot and channel
//     (zero when the slot was taken) and is moved on by the step's tokens.  The gates, the
//     candidate and the recurrence are float32; y is stored in the activation type.
//     The recurrence is linear in S, S_t = a_t S_(t-1) + b_t, so a sequence's tokens are cut into
//     as many segments as the block has warps: every warp first composes its segment into one
//     pair (A, B) from a zero start, a thread per channel chains the pairs of the segments before
//     its own onto the slot's state, and the warp walks its segment again from there.
// bfi_bias_act: y[t, j] = act(u[t, j] + b[j]) (tanh GELU), and, when asked, fill[t, :] = b2, the
//     bias of the product that follows and accumulates into those float32 rows.
// bfi_sigmoid_gate: x[t, j] *= sigmoid(g[t, j / group]) over rows of the activation type: one gate
//     per value (group 1) or per head (group = the head's size).
#include "common.cuh"

#define SCAN_CAND_IDENTITY 0
#define SCAN_CAND_POSITIVE 1
#define SCAN_MAX_WARPS 32

__device__ __forceinline__ float cw_sigmoid(float x) {
    if (x >= 0.0f) return 1.0f / (1.0f + expf(-x));
    const float z = expf(x);
    return z / (1.0f + z);
}

struct ScanArgs {
    long p_stride, y_stride;
    int z_off, u_off, g_off;        // g_off < 0: no output gate
    int C, cand, tiles;
    const float *z_bias, *u_bias;   // float32 [C] or null
    const int *cu_seqlens, *seq_slot;
};

// float32 arithmetic in both; with bfloat16 projections the exponential and the division are the hardware's
// approximations (a few units in the last place of a float32, far below what the projections' rounding left)
template <typename T>
__device__ __forceinline__ float scan_sigmoid(float x) { return cw_sigmoid(x); }
template <>
__device__ __forceinline__ float scan_sigmoid<bf16>(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

template <typename T>
__device__ __forceinline__ void scan_coefficients(float z_raw, float u_raw, int cand_kind, float bz, float bu, float& keep,
                                                  float& add) {
    const float z = scan_sigmoid<T>(z_raw + bz);
    const float u = u_raw + bu;
    const float cand = cand_kind == SCAN_CAND_POSITIVE ? (u >= 0.0f ? u + 0.5f : scan_sigmoid<T>(u)) : u;
    keep = 1.0f - z;
    add = z * cand;
}

#define SCAN_UNROLL 8       // tokens whose inputs are in flight before the chain of multiply-adds walks them

template <typename T>
__global__ void __launch_bounds__(32 * SCAN_MAX_WARPS)
gated_scan_kernel(const T* __restrict__ proj, T* __restrict__ y, float* __restrict__ state, const ScanArgs a) {
    pdl_trigger();
    __shared__ float seg_a[SCAN_MAX_WARPS][32], seg_b[SCAN_MAX_WARPS][32];
    const int seq = blockIdx.x;
    // a.tiles > 1 (steps whose sequences bring few tokens): the block's warps are channel tiles of one segment each
    const int lane = threadIdx.x;
    const int w = a.tiles > 1 ? 0 : threadIdx.y, n_w = a.tiles > 1 ? 1 : blockDim.y;
    const int ch = (a.tiles > 1 ? blockIdx.y * a.tiles + threadIdx.y : blockIdx.y) * 32 + lane;
    const bool live = ch < a.C;
    const float bz = (live && a.z_bias) ? a.z_bias[ch] : 0.0f;
    const float bu = (live && a.u_bias) ? a.u_bias[ch] : 0.0f;
    pdl_wait();
    const int slot = a.seq_slot[seq];
    if (slot < 0) return;
    const int t0 = a.cu_seqlens[seq], nt = a.cu_seqlens[seq + 1] - t0;
    const int per = (nt + n_w - 1) / n_w;
    const int first = min(nt, w * per), last = min(nt, first + per);
    const T* base = proj + (size_t)t0 * a.p_stride + ch;
    float A = 1.0f, B = 0.0f;
    if (n_w > 1 && live) {
        for (int t = first; t < last; t += SCAN_UNROLL) {
            float zr[SCAN_UNROLL], ur[SCAN_UNROLL];
#pragma unroll
            for (int i = 0; i < SCAN_UNROLL; ++i) {
                const T* row = base + (size_t)min(t + i, last - 1) * a.p_stride;
                zr[i] = to_f32(row[a.z_off]);
                ur[i] = to_f32(row[a.u_off]);
            }
#pragma unroll
            for (int i = 0; i < SCAN_UNROLL; ++i) {
                if (t + i < last) {
                    float keep, add;
                    scan_coefficients<T>(zr[i], ur[i], a.cand, bz, bu, keep, add);
                    B = fmaf(keep, B, add);
                    A *= keep;
                }
            }
        }
    }
    if (n_w > 1) {
        seg_a[w][lane] = A;
        seg_b[w][lane] = B;
        __syncthreads();
    }
    if (!live) return;
    float S = state[(size_t)slot * a.C + ch];
    for (int i = 0; i < w; ++i) S = fmaf(seg_a[i][lane], S, seg_b[i][lane]);
    for (int t = first; t < last; t += SCAN_UNROLL) {
        float zr[SCAN_UNROLL], ur[SCAN_UNROLL], gr[SCAN_UNROLL];
#pragma unroll
        for (int i = 0; i < SCAN_UNROLL; ++i) {
            const T* row = base + (size_t)min(t + i, last - 1) * a.p_stride;
            zr[i] = to_f32(row[a.z_off]);
            ur[i] = to_f32(row[a.u_off]);
            gr[i] = a.g_off >= 0 ? to_f32(row[a.g_off]) : 0.0f;
        }
#pragma unroll
        for (int i = 0; i < SCAN_UNROLL; ++i) {
            if (t + i < last) {
                float keep, add;
                scan_coefficients<T>(zr[i], ur[i], a.cand, bz, bu, keep, add);
                S = fmaf(keep, S, add);
                float out = S;
                if (a.g_off >= 0) out *= gr[i] * scan_sigmoid<T>(gr[i]);
                y[(size_t)(t0 + t + i) * a.y_stride + ch] = from_f32<T>(out);
            }
        }
    }
    if (w == n_w - 1) state[(size_t)slot * a.C + ch] = S;     // the last warp's end is the sequence's
}

extern "C" int bfi_gated_scan(const void* proj, long p_stride, int z_off, int u_off, int g_off, int dtype, const float* z_bias,
                              const float* u_bias, void* y, long y_stride, float* state, const int* cu_seqlens,
                              const int* seq_slot, int n_seqs, int C, int cand, int max_seq_tokens, cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(dtype), "gated_scan: unknown dtype code %d", dtype);
    BFI_REQUIRE(C > 0 && z_off >= 0 && u_off >= 0, "gated_scan: bad sizes channels=%d", C);
    BFI_REQUIRE(cand == SCAN_CAND_IDENTITY || cand == SCAN_CAND_POSITIVE, "gated_scan: unknown candidate kind %d", cand);
    BFI_REQUIRE(p_stride >= z_off + C && p_stride >= u_off + C && p_stride >= g_off + C && y_stride >= C,
                "gated_scan: row stride shorter than the channels");
    if (n_seqs <= 0) return 0;
    int warps = (max_seq_tokens + 15) / 16;        // segments of at least 16 tokens, as many as a block has warps
    if (warps < 1) warps = 1;
    if (warps > SCAN_MAX_WARPS) warps = SCAN_MAX_WARPS;
    const int tiles = warps == 1 ? 4 : 1;          // one segment: four channel tiles share a block
    const dim3 grid(n_seqs, ((C + 31) / 32 + tiles - 1) / tiles), block(32, warps == 1 ? tiles : warps);
    BFI_REQUIRE(grid.y <= 65535, "gated_scan: %d channels are too many for one launch", C);
    ScanArgs a;
    a.p_stride = p_stride, a.y_stride = y_stride, a.z_off = z_off, a.u_off = u_off, a.g_off = g_off, a.C = C, a.cand = cand, a.tiles = tiles;
    a.z_bias = z_bias, a.u_bias = u_bias, a.cu_seqlens = cu_seqlens, a.seq_slot = seq_slot;
    if (dtype == BFI_F32)
        bfi_launch(gated_scan_kernel<float>, grid, block, 0, stream, (const float*)proj, (float*)y, state, a);
    else
        bfi_launch(gated_scan_kernel<bf16>, grid, block, 0, stream, (const bf16*)proj, (bf16*)y, state, a);
    return bfi_check_launch("gated_scan");
}

// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void bias_act_kernel(const T* __restrict__ u, long u_stride, const void* __restrict__ bias, int b_dtype,
                                T* __restrict__ y, long y_stride, int cols, float* __restrict__ fill, long fill_stride,
                                const void* __restrict__ fill_bias, int fb_dtype, int fill_cols) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.y;
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j < cols) {
        float v = to_f32(u[(size_t)t * u_stride + j]);
        if (bias) v += load_as_f32(bias, b_dtype, j);
        y[(size_t)t * y_stride + j] = from_f32<T>(gelu_tanh_exact(v));
    }
    if (fill != nullptr && j < fill_cols) fill[(size_t)t * fill_stride + j] = load_as_f32(fill_bias, fb_dtype, j);
}

// 0.5 z (1 + tanh(y)) = z * sigmoid(2 y), with the hardware's exponential and division (the matrix products' gated
// epilogue evaluates it the same way for bfloat16)
__device__ __forceinline__ float gelu_tanh_fast(float g) {
    const float y = 0.7978845608028654f * (g + 0.044715f * g * g * g);
    return __fdividef(g, 1.0f + __expf(-2.0f * y));
}

// bfloat16 rows whose columns come in whole groups of 8: a thread takes 16 bytes of a row (and, of the rows to
// fill, the 8 float32 values at the same columns, in as many turns as the wider of the two needs)
__global__ void bias_act_vec_kernel(const bf16* __restrict__ u, long u_stride, const void* __restrict__ bias, int b_dtype,
                                    bf16* __restrict__ y, long y_stride, int cols, float* __restrict__ fill, long fill_stride,
                                    const void* __restrict__ fill_bias, int fb_dtype, int fill_cols, int n_rows) {
    pdl_trigger();
    pdl_wait();
    const bool bias_vec = b_dtype == BFI_BF16 && (reinterpret_cast<uintptr_t>(bias) & 15) == 0;
    const int groups = cols >> 3, fill_groups = fill != nullptr ? fill_cols >> 3 : 0;
    const int per_row = groups > fill_groups ? groups : fill_groups;
    const long total = (long)n_rows * per_row;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const int t = (int)(i / per_row), gq = (int)(i - (long)t * per_row);
        const int j = gq << 3;
        if (gq < groups) {
            const uint4 raw = *reinterpret_cast<const uint4*>(u + (size_t)t * u_stride + j);
            const __nv_bfloat162* in = reinterpret_cast<const __nv_bfloat162*>(&raw);
            uint4 packed;
            __nv_bfloat162* out = reinterpret_cast<__nv_bfloat162*>(&packed);
            float b8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (bias && bias_vec) {                // 16 bytes of a bfloat16 bias at once
                const uint4 braw = *reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(bias) + j);
                const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&braw);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 f = __bfloat1622float2(bh[k]);
                    b8[2 * k] = f.x, b8[2 * k + 1] = f.y;
                }
            } else if (bias) {
#pragma unroll
                for (int k = 0; k < 8; ++k) b8[k] = load_as_f32(bias, b_dtype, j + k);
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float2 v = __bfloat1622float2(in[k]);
                v.x += b8[2 * k];
                v.y += b8[2 * k + 1];
                out[k] = __floats2bfloat162_rn(gelu_tanh_fast(v.x), gelu_tanh_fast(v.y));
            }
            *reinterpret_cast<uint4*>(y + (size_t)t * y_stride + j) = packed;
        }
        if (gq < fill_groups) {
            float4 a, b;
            a.x = load_as_f32(fill_bias, fb_dtype, j), a.y = load_as_f32(fill_bias, fb_dtype, j + 1);
            a.z = load_as_f32(fill_bias, fb_dtype, j + 2), a.w = load_as_f32(fill_bias, fb_dtype, j + 3);
            b.x = load_as_f32(fill_bias, fb_dtype, j + 4), b.y = load_as_f32(fill_bias, fb_dtype, j + 5);
            b.z = load_as_f32(fill_bias, fb_dtype, j + 6), b.w = load_as_f32(fill_bias, fb_dtype, j + 7);
            float4* dst = reinterpret_cast<float4*>(fill + (size_t)t * fill_stride + j);
            dst[0] = a;
            dst[1] = b;
        }
    }
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

extern "C" int bfi_bias_act(const void* u, long u_stride, int dtype, const void* bias, int b_dtype, void* y, long y_stride,
                            int n_rows, int cols, float* fill, long fill_stride, const void* fill_bias, int fb_dtype,
                            int fill_cols, cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(dtype) && dtype_ok(b_dtype) && dtype_ok(fb_dtype), "bias_act: unknown dtype code");
    BFI_REQUIRE(n_rows >= 0 && cols > 0 && u_stride >= cols && y_stride >= cols, "bias_act: bad sizes rows=%d cols=%d", n_rows, cols);
    BFI_REQUIRE(fill == nullptr || (fill_bias != nullptr && fill_cols > 0 && fill_stride >= fill_cols),
                "bias_act: the rows to fill need their bias and a stride of their width");
    if (n_rows == 0) return 0;
    const int widest = (fill != nullptr && fill_cols > cols) ? fill_cols : cols;
    if (dtype == BFI_BF16 && cols % 8 == 0 && u_stride % 8 == 0 && y_stride % 8 == 0 && aligned16(u) && aligned16(y) &&
        (fill == nullptr || (fill_cols % 8 == 0 && fill_stride % 4 == 0 && aligned16(fill)))) {
        const long total = (long)n_rows * (widest / 8);
        long blocks = (total + 255) / 256;
        const long most = (long)bfi_sm_count() * 16;
        if (blocks > most) blocks = most;
        bfi_launch(bias_act_vec_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, (const bf16*)u, u_stride, bias, b_dtype, (bf16*)y,
                   y_stride, cols, fill, fill_stride, fill_bias, fb_dtype, fill_cols, n_rows);
        return bfi_check_launch("bias_act");
    }
    BFI_REQUIRE(n_rows <= 65535, "bias_act: %d rows are too many for one launch", n_rows);
    const dim3 grid((widest + 255) / 256, n_rows);
    if (dtype == BFI_F32)
        bfi_launch(bias_act_kernel<float>, grid, dim3(256), 0, stream, (const float*)u, u_stride, bias, b_dtype, (float*)y, y_stride,
                   cols, fill, fill_stride, fill_bias, fb_dtype, fill_cols);
    else
        bfi_launch(bias_act_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16*)u, u_stride, bias, b_dtype, (bf16*)y, y_stride,
                   cols, fill, fill_stride, fill_bias, fb_dtype, fill_cols);
    return bfi_check_launch("bias_act");
}

// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ x, long x_stride, const T* __restrict__ g, long g_stride, int cols, int group) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.y;
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= cols) return;
    T* p = x + (size_t)t * x_stride + j;
    *p = from_f32<T>(to_f32(*p) * cw_sigmoid(to_f32(g[(size_t)t * g_stride + j / group])));
}

// bfloat16 rows in whole groups of 8 values that share a gate or have one each
__global__ void sigmoid_gate_vec_kernel(bf16* __restrict__ x, long x_stride, const bf16* __restrict__ g, long g_stride, int cols,
                                        int group, int n_rows) {
    pdl_trigger();
    pdl_wait();
    const int per_row = cols >> 3;
    const long total = (long)n_rows * per_row;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const int t = (int)(i / per_row), j = (int)(i - (long)t * per_row) << 3;
        uint4 raw = *reinterpret_cast<const uint4*>(x + (size_t)t * x_stride + j);
        __nv_bfloat162* v = reinterpret_cast<__nv_bfloat162*>(&raw);
        float gate[8];
        if (group == 1) {
            const uint4 graw = *reinterpret_cast<const uint4*>(g + (size_t)t * g_stride + j);
            const __nv_bfloat162* gv = reinterpret_cast<const __nv_bfloat162*>(&graw);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 f = __bfloat1622float2(gv[k]);
                gate[2 * k] = f.x, gate[2 * k + 1] = f.y;
            }
        } else {                                   // the 8 values lie in one group
            const float one = __bfloat162float(g[(size_t)t * g_stride + j / group]);
#pragma unroll
            for (int k = 0; k < 8; ++k) gate[k] = one;
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 f = __bfloat1622float2(v[k]);
            v[k] = __floats2bfloat162_rn(__fdividef(f.x, 1.0f + __expf(-gate[2 * k])), __fdividef(f.y, 1.0f + __expf(-gate[2 * k + 1])));
        }
        *reinterpret_cast<uint4*>(x + (size_t)t * x_stride + j) = raw;
    }
}

extern "C" int bfi_sigmoid_gate(void* x, long x_stride, const void* g, long g_stride, int dtype, int n_rows, int cols, int group,
                                cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(dtype), "sigmoid_gate: unknown dtype code %d", dtype);
    BFI_REQUIRE(n_rows >= 0 && cols > 0 && group > 0 && cols % group == 0 && x_stride >= cols && g_stride >= cols / group,
                "sigmoid_gate: bad sizes rows=%d cols=%d group=%d", n_rows, cols, group);
    if (n_rows == 0) return 0;
    if (dtype == BFI_BF16 && cols % 8 == 0 && x_stride % 8 == 0 && aligned16(x) && (group % 8 == 0 || (group == 1 && g_stride % 8 == 0 && aligned16(g)))) {
        const long total = (long)n_rows * (cols / 8);
        long blocks = (total + 255) / 256;
        const long most = (long)bfi_sm_count() * 16;
        if (blocks > most) blocks = most;
        bfi_launch(sigmoid_gate_vec_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, (bf16*)x, x_stride, (const bf16*)g, g_stride, cols,
                   group, n_rows);
        return bfi_check_launch("sigmoid_gate");
    }
    BFI_REQUIRE(n_rows <= 65535, "sigmoid_gate: %d rows are too many for one launch", n_rows);
    const dim3 grid((cols + 255) / 256, n_rows);
    if (dtype == BFI_F32)
        bfi_launch(sigmoid_gate_kernel<float>, grid, dim3(256), 0, stream, (float*)x, x_stride, (const float*)g, g_stride, cols, group);
    else
        bfi_launch(sigmoid_gate_kernel<bf16>, grid, dim3(256), 0, stream, (bf16*)x, x_stride, (const bf16*)g, g_stride, cols, group);
    return bfi_check_launch("sigmoid_gate");
}

BFI_TRACE_EXPORT(channelwise)
