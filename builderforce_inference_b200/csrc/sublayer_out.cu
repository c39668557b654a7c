// What happens to a sublayer's output on its way into the residual stream when the block does more
// than add it: a norm of the output before the add, and a weighted sum of two outputs.
//
//   bfi_norm_add:      x[t, :] += mult * y'[t, :] * rsqrt(mean(y'[t, :]^2) + eps) * w   (y float32)
//                      with y' = y, or, given gate logits g (and a bias b), y' = y * sigmoid(g + b)
//                      and, in single-token steps when asked, the convolution over time in front of the next sublayer
//                      on the row just made (see ConvTail);
//                      and, when asked, the next sublayer's norm of the new x in the same kernel:
//                      h[t, :] = x[t, :] * rsqrt(mean(x[t, :]^2) + eps2) * w2       (h in the activation dtype)
//   bfi_weighted_sum:  out[t, :] = a * y0[t, :] + b * y1[t, :]                      (all float32)
//   bfi_scale_rows:    x[r, :] *= s                                                 (float32)
//   bfi_gated_rows:    out[r, :] (= | +=) g[r] * src[r, :]                          (float32)
//
// The residual stream x and the sublayer outputs are float32 in every run dtype; the weight is
// float32 or bfloat16.  All arithmetic is float32.
#include "common.cuh"

struct NormAddGate {
    const void* logits;       // null: no gate
    int dtype;
    long stride;
    const void* bias;         // null: none
    int bias_dtype;
};

__device__ __forceinline__ float out_sigmoid(float x) {
    if (x >= 0.0f) return 1.0f / (1.0f + expf(-x));
    const float z = expf(x);
    return z / (1.0f + z);
}

__global__ void norm_add_kernel(float* __restrict__ x, long x_stride, const float* __restrict__ y, long y_stride,
                                const void* __restrict__ w, int w_dtype, int width, float eps, const void* __restrict__ w2,
                                int w2_dtype, float eps2, void* __restrict__ h, int h_dtype, long h_stride, float mult,
                                const NormAddGate g) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const float* yr = y + (size_t)t * y_stride;
    float* xr = x + (size_t)t * x_stride;
    const bool gated = g.logits != nullptr;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        float v = yr[j];
        if (gated) {
            float z = load_as_f32(g.logits, g.dtype, (size_t)t * g.stride + j);
            if (g.bias) z += load_as_f32(g.bias, g.bias_dtype, j);
            v *= out_sigmoid(z);
        }
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    float ss2 = 0.0f;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        float yv = yr[j];
        if (gated) {
            float z = load_as_f32(g.logits, g.dtype, (size_t)t * g.stride + j);
            if (g.bias) z += load_as_f32(g.bias, g.bias_dtype, j);
            yv *= out_sigmoid(z);
        }
        const float v = xr[j] + mult * (yv * scale * load_as_f32(w, w_dtype, j));
        xr[j] = v;
        ss2 = fmaf(v, v, ss2);
    }
    if (h == nullptr) return;
    ss2 = block_sum(ss2, scratch);
    const float scale2 = 1.0f / sqrtf(ss2 / (float)width + eps2);
    // every thread reads back the values it wrote itself
    for (int j = threadIdx.x; j < width; j += blockDim.x)
        store_from_f32(h, h_dtype, (size_t)t * h_stride + j, xr[j] * scale2 * load_as_f32(w2, w2_dtype, j));
}

// The same for rows of a multiple of 4 values: a thread keeps its share of the gated row, and then of the new x, in
// registers, so y, the gate's logits and x are read once.
__device__ __forceinline__ float4 load4_as_f32(const void* p, int dtype, size_t i) {      // i a multiple of 4, p aligned for it
    if (dtype == BFI_F32) return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
    const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const bf16*>(p) + i);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float2 a = __bfloat1622float2(h2[0]), b = __bfloat1622float2(h2[1]);
    return make_float4(a.x, a.y, b.x, b.y);
}

// What may follow the add in a step in which every sequence brings one token: the convolution over time that stands in
// front of the NEXT sublayer (2 to 4 taps, no bias), on the row just made.  With the new x as the current input and the
// slot's kept inputs as the earlier ones,
//     h[t, c] = x[t, c] + sum_j w[c, taps-1-j] in_j[c]          plain[t, c] = x[t, c]
// both in the activation type, and the kept inputs move on by one.  A thread owns its channels of the row in both
// parts, so nothing is read by another thread between them.
struct ConvTail {
    const void* w;            // null: no tail
    int w_dtype, taps;
    float* state;             // [slots][taps-1][width]
    const int* token_slot;
    void* h;
    long h_stride;
    void* plain;
    long plain_stride;
    int out_dtype;
};

__device__ __forceinline__ void store4_from_f32(void* p, int dtype, size_t i, const float4 v) {
    if (dtype == BFI_F32) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + i) = v;
    } else {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        uint2 packed;
        packed.x = *reinterpret_cast<const uint32_t*>(&lo);
        packed.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(p) + i) = packed;
    }
}

__device__ __forceinline__ void conv_tail_chunk(const ConvTail& ct, int t, int slot, int width, int c, const float4 cur) {
    const int taps = ct.taps;
    float* st = ct.state + (size_t)slot * (taps - 1) * width + c;
    float4 kept[3];                                // the inputs 1, 2, 3 steps back (taps <= 4)
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    const float in0[4] = {cur.x, cur.y, cur.z, cur.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) acc[k] = fmaf(load_as_f32(ct.w, ct.w_dtype, (size_t)(c + k) * taps + (taps - 1)), in0[k], acc[k]);
#pragma unroll
    for (int j = 1; j < 4; ++j) {
        if (j < taps) {
            kept[j - 1] = *reinterpret_cast<const float4*>(st + (size_t)(taps - 1 - j) * width);
            const float in[4] = {kept[j - 1].x, kept[j - 1].y, kept[j - 1].z, kept[j - 1].w};
#pragma unroll
            for (int k = 0; k < 4; ++k)
                acc[k] = fmaf(load_as_f32(ct.w, ct.w_dtype, (size_t)(c + k) * taps + (taps - 1 - j)), in[k], acc[k]);
        }
    }
    store4_from_f32(ct.h, ct.out_dtype, (size_t)t * ct.h_stride + c, make_float4(acc[0] + in0[0], acc[1] + in0[1], acc[2] + in0[2], acc[3] + in0[3]));
    store4_from_f32(ct.plain, ct.out_dtype, (size_t)t * ct.plain_stride + c, cur);
    // the window moves on by one: the input j steps back takes the place of the one j + 1 steps back
    *reinterpret_cast<float4*>(st + (size_t)(taps - 2) * width) = cur;
#pragma unroll
    for (int j = 1; j < 3; ++j)
        if (j < taps - 1) *reinterpret_cast<float4*>(st + (size_t)(taps - 2 - j) * width) = kept[j - 1];
}

// EARLY (few rows: a single-token step): the weights before the wait for the kernel before this one, and x asked for
// together with y and the gate's logits, so the row costs one trip to memory instead of two; with many rows the
// registers that takes cost more in resident rows than the trip does.
template <int VPT, bool EARLY>
__global__ void __launch_bounds__(256)
norm_add_vec_kernel(float* __restrict__ x, long x_stride, const float* __restrict__ y, long y_stride, const void* __restrict__ w,
                    int w_dtype, int width, float eps, float mult, const NormAddGate g, const void* __restrict__ w2, int w2_dtype,
                    float eps2, void* __restrict__ h, int h_dtype, long h_stride, const ConvTail ct) {
    pdl_trigger();
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const int n4 = width >> 2;
    // the weights and the gate's bias do not come from the kernel before this one: fetched before the wait
    float4 wv[EARLY ? VPT : 1];
    if (EARLY) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int j = i * 256 + threadIdx.x;
            wv[i] = j < n4 ? load4_as_f32(w, w_dtype, (size_t)j * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    pdl_wait();
    const float4* yr = reinterpret_cast<const float4*>(y + (size_t)t * y_stride);
    float4* xr = reinterpret_cast<float4*>(x + (size_t)t * x_stride);
    float4 v[VPT], xv[EARLY ? VPT : 1];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int j = i * 256 + threadIdx.x;
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (j < n4) {
            v[i] = yr[j];
            if (EARLY) xv[i] = xr[j];
        }
    }
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int j = i * 256 + threadIdx.x;
        if (j >= n4) continue;
        if (g.logits != nullptr) {
            float4 z = load4_as_f32(g.logits, g.dtype, (size_t)t * g.stride + (size_t)j * 4);
            if (g.bias != nullptr) {
                const float4 b = load4_as_f32(g.bias, g.bias_dtype, (size_t)j * 4);
                z.x += b.x, z.y += b.y, z.z += b.z, z.w += b.w;
            }
            v[i].x *= out_sigmoid(z.x);
            v[i].y *= out_sigmoid(z.y);
            v[i].z *= out_sigmoid(z.z);
            v[i].w *= out_sigmoid(z.w);
        }
        ss = fmaf(v[i].x, v[i].x, ss);
        ss = fmaf(v[i].y, v[i].y, ss);
        ss = fmaf(v[i].z, v[i].z, ss);
        ss = fmaf(v[i].w, v[i].w, ss);
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int j = i * 256 + threadIdx.x;
        if (j >= n4) continue;
        float4 o = EARLY ? xv[i] : xr[j];
        const float4 ww = EARLY ? wv[i] : load4_as_f32(w, w_dtype, (size_t)j * 4);
        o.x += mult * (v[i].x * scale * ww.x);
        o.y += mult * (v[i].y * scale * ww.y);
        o.z += mult * (v[i].z * scale * ww.z);
        o.w += mult * (v[i].w * scale * ww.w);
        xr[j] = o;
        v[i] = o;
    }
    if (ct.w != nullptr) {
        const int slot = ct.token_slot[t];
        if (slot >= 0) {
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int j = i * 256 + threadIdx.x;
                if (j < n4) conv_tail_chunk(ct, t, slot, width, j * 4, v[i]);
            }
        }
    }
    if (h == nullptr) return;
    float ss2 = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        if (i * 256 + threadIdx.x >= n4) continue;
        ss2 = fmaf(v[i].x, v[i].x, ss2);
        ss2 = fmaf(v[i].y, v[i].y, ss2);
        ss2 = fmaf(v[i].z, v[i].z, ss2);
        ss2 = fmaf(v[i].w, v[i].w, ss2);
    }
    ss2 = block_sum(ss2, scratch);
    const float scale2 = 1.0f / sqrtf(ss2 / (float)width + eps2);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int j = i * 256 + threadIdx.x;
        if (j >= n4) continue;
        const int c = j * 4;
        const size_t at = (size_t)t * h_stride + c;
        store_from_f32(h, h_dtype, at, v[i].x * scale2 * load_as_f32(w2, w2_dtype, c));
        store_from_f32(h, h_dtype, at + 1, v[i].y * scale2 * load_as_f32(w2, w2_dtype, c + 1));
        store_from_f32(h, h_dtype, at + 2, v[i].z * scale2 * load_as_f32(w2, w2_dtype, c + 2));
        store_from_f32(h, h_dtype, at + 3, v[i].w * scale2 * load_as_f32(w2, w2_dtype, c + 3));
    }
}

extern "C" int bfi_norm_add(float* x, long x_stride, const float* y, long y_stride, const void* w, int w_dtype,
                            int n_rows, int width, float eps, const void* w2, int w2_dtype, float eps2, void* h,
                            int h_dtype, long h_stride, float mult, const void* gate, int gate_dtype, long gate_stride,
                            const void* gate_bias, int gate_bias_dtype, const void* conv_w, int conv_w_dtype, int conv_taps,
                            float* conv_state, const int* token_slot, void* conv_h, long conv_h_stride, void* conv_plain,
                            long conv_plain_stride, int conv_out_dtype, cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(w_dtype) && dtype_ok(w2_dtype) && dtype_ok(h_dtype) && dtype_ok(gate_dtype) && dtype_ok(gate_bias_dtype),
                "norm_add: unknown dtype code");
    BFI_REQUIRE(n_rows >= 0 && width > 0, "norm_add: bad sizes rows=%d width=%d", n_rows, width);
    BFI_REQUIRE(x_stride >= width && y_stride >= width, "norm_add: row stride shorter than the row");
    BFI_REQUIRE(h == nullptr || (w2 != nullptr && h_stride >= width), "norm_add: the next norm needs its weight and rows of the width");
    BFI_REQUIRE(gate == nullptr || gate_stride >= width, "norm_add: the gate's row stride is shorter than the row");
    if (n_rows == 0) return 0;
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    ConvTail ct;
    ct.w = conv_w, ct.w_dtype = conv_w_dtype, ct.taps = conv_taps, ct.state = conv_state, ct.token_slot = token_slot;
    ct.h = conv_h, ct.h_stride = conv_h_stride, ct.plain = conv_plain, ct.plain_stride = conv_plain_stride, ct.out_dtype = conv_out_dtype;
    if (conv_w != nullptr) {
        BFI_REQUIRE(dtype_ok(conv_w_dtype) && dtype_ok(conv_out_dtype), "norm_add: unknown dtype code of the convolution that follows");
        BFI_REQUIRE(conv_taps >= 2 && conv_taps <= 4 && conv_state != nullptr && token_slot != nullptr && conv_h != nullptr &&
                        conv_plain != nullptr && conv_h_stride >= width && conv_plain_stride >= width,
                    "norm_add: the convolution that follows takes 2 to 4 taps, its state, the tokens' slots and two outputs of the width");
    }
    NormAddGate g;
    g.logits = gate, g.dtype = gate_dtype, g.stride = gate_stride, g.bias = gate != nullptr ? gate_bias : nullptr;
    g.bias_dtype = gate_bias_dtype;
    const auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    // the plain normed add keeps the kernel (and with it the order of its sums) it has always had
    const auto al_for = [](const void* p, int dt) { return (reinterpret_cast<uintptr_t>(p) & (dt == BFI_F32 ? 15 : 7)) == 0; };
    const auto al_out = [](const void* p, long stride, int dt) {
        return (reinterpret_cast<uintptr_t>(p) & (dt == BFI_F32 ? 15 : 7)) == 0 && stride % 4 == 0;
    };
    const bool tail_ok = conv_w == nullptr || (al_out(conv_h, conv_h_stride, conv_out_dtype) && al_out(conv_plain, conv_plain_stride, conv_out_dtype) &&
                                               (reinterpret_cast<uintptr_t>(conv_state) & 15) == 0);
    if ((gate != nullptr || mult != 1.0f || conv_w != nullptr) && tail_ok && al_for(w, w_dtype) && (gate_bias == nullptr || al_for(gate_bias, gate_bias_dtype)) && width % 4 == 0 &&
        width <= 8 * 4 * 256 && x_stride % 4 == 0 && y_stride % 4 == 0 && al16(x) && al16(y) &&
        (gate == nullptr || (gate_stride % 4 == 0 && (((uintptr_t)gate) & (gate_dtype == BFI_F32 ? 15 : 7)) == 0))) {
        const int vpt = (width / 4 + 255) / 256;
        const bool early = n_rows <= 2 * bfi_sm_count();
#define BFI_NORM_ADD(V)                                                                                                    \
    do {                                                                                                                     \
    if (early)                                                                                                               \
        bfi_launch(norm_add_vec_kernel<V, true>, dim3(n_rows), dim3(256), 0, stream, x, x_stride, y, y_stride, w, w_dtype, width, \
                   eps, mult, g, w2, w2_dtype, eps2, h, h_dtype, h_stride, ct);                                              \
    else                                                                                                                     \
        bfi_launch(norm_add_vec_kernel<V, false>, dim3(n_rows), dim3(256), 0, stream, x, x_stride, y, y_stride, w, w_dtype, width, \
                   eps, mult, g, w2, w2_dtype, eps2, h, h_dtype, h_stride, ct);                                              \
    } while (0)
        if (vpt <= 1) BFI_NORM_ADD(1);
        else if (vpt == 2) BFI_NORM_ADD(2);
        else if (vpt <= 4) BFI_NORM_ADD(4);
        else BFI_NORM_ADD(8);
#undef BFI_NORM_ADD
        return bfi_check_launch("norm_add");
    }
    BFI_REQUIRE(conv_w == nullptr, "norm_add: the convolution that follows needs rows of a multiple of 4 values (at most 8192) on 16-byte borders");
    bfi_launch(norm_add_kernel, dim3(n_rows), dim3(threads), 0, stream, x, x_stride, y, y_stride, w, w_dtype, width, eps, w2,
               w2_dtype, eps2, h, h_dtype, h_stride, mult, g);
    return bfi_check_launch("norm_add");
}

__global__ void weighted_sum_kernel(float* __restrict__ out, const float* __restrict__ y0, float a,
                                    const float* __restrict__ y1, float b, long n) {
    pdl_trigger();
    pdl_wait();
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = a * y0[i] + b * y1[i];
}

extern "C" int bfi_weighted_sum(float* out, const float* y0, float a, const float* y1, float b, long n,
                                cudaStream_t stream) {
    BFI_REQUIRE(n >= 0, "weighted_sum: negative size");
    if (n == 0) return 0;
    bfi_launch(weighted_sum_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, out, y0, a, y1, b, n);
    return bfi_check_launch("weighted_sum");
}

__global__ void scale_rows_kernel(float* __restrict__ x, long stride, int cols, float s) {
    pdl_trigger();
    pdl_wait();
    float* r = x + (size_t)blockIdx.y * stride;
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j < cols) r[j] *= s;
}

// x[r, :] *= s over float32 rows (the logits' scale)
extern "C" int bfi_scale_rows(float* x, long stride, int n_rows, int cols, float s, cudaStream_t stream) {
    BFI_REQUIRE(n_rows >= 0 && cols > 0 && stride >= cols, "scale_rows: bad sizes rows=%d cols=%d", n_rows, cols);
    if (n_rows == 0) return 0;
    BFI_REQUIRE(n_rows <= 65535, "scale_rows: %d rows are too many for one launch", n_rows);
    bfi_launch(scale_rows_kernel, dim3((cols + 255) / 256, n_rows), dim3(256), 0, stream, x, stride, cols, s);
    return bfi_check_launch("scale_rows");
}

__global__ void gated_rows_kernel(float* __restrict__ out, long out_stride, const float* __restrict__ src, long src_stride,
                                  const float* __restrict__ g, int cols, int accumulate) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.y;
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= cols) return;
    float* o = out + (size_t)r * out_stride + j;
    const float v = g[r] * src[(size_t)r * src_stride + j];
    *o = accumulate ? *o + v : v;
}

// out[r, :] (= | +=) g[r] * src[r, :] over float32 rows (a sublayer's part with one factor per token)
extern "C" int bfi_gated_rows(float* out, long out_stride, const float* src, long src_stride, const float* g, int n_rows,
                              int cols, int accumulate, cudaStream_t stream) {
    BFI_REQUIRE(n_rows >= 0 && cols > 0 && out_stride >= cols && src_stride >= cols, "gated_rows: bad sizes rows=%d cols=%d", n_rows, cols);
    if (n_rows == 0) return 0;
    BFI_REQUIRE(n_rows <= 65535, "gated_rows: %d rows are too many for one launch", n_rows);
    bfi_launch(gated_rows_kernel, dim3((cols + 255) / 256, n_rows), dim3(256), 0, stream, out, out_stride, src, src_stride, g, cols,
               accumulate);
    return bfi_check_launch("gated_rows");
}

BFI_TRACE_EXPORT(sublayer_out)
