// A routed feed-forward (mixture of experts): the router's decision and the experts' products for
// the (token, chosen expert) pairs, reading only the chosen experts' weights.  Float32 or
// bfloat16 storage of activations and expert weights, float32 arithmetic everywhere.
//
// bfi_moe_route, per token with router logits z[0..E) (float32):
//     s = softmax(z);  choice_e = s_e + correction_e
//     experts form `n_groups` equal groups of neighbours; a group's score is its largest choice
//     score; only experts of the `keep` best groups can be chosen (the others count as minus
//     infinity); the `top` largest choice scores among them are chosen, the lowest index winning
//     a tie; the weights are the chosen experts' s (not renormalised) times `weight_scale`.
//     With `extra` (a logit beside the experts', column E of z) gate[t] = sigmoid(z_E): the factor
//     of an expert that every token uses.
//     `score_mode` 1: s = sigmoid(z), every expert by itself, instead of the softmax.
//     `group_top` g > 1: a group's score is the sum of its g largest choice scores (of all of them,
//     if it has fewer) instead of the largest.
// `act_kind` of the experts: 0 = silu(gate) * up over interleaved gate and up rows (W_gu as below);
//     1 = relu(up)^2, no gate: W_gu is then [E * ff, width], expert e's up row j at row e ff + j.
// bfi_moe_router: the same decision with the logits made here, z = W_router h (float32 rows of W).
// bfi_moe_gate_up:  act[t, k, :] = silu(W_gate[e] h_t) * (W_up[e] h_t),  e = idx[t, k]
// bfi_moe_down:     out[t, :] (= | +=) sum_k weight[t, k] * W_down[idx[t, k]] act[t, k, :]
//                                      + gate[t] * shared[t, :]            (the last term optional)
// The experts' weights are two matrices for all experts, the layouts the dense products take as well:
// W_gu [E * 2 * ff, width], expert e's gate row j at row 2 (e ff + j) and its up row right after it;
// W_down [width, E * ff], expert e's columns at e ff .. (e + 1) ff.
// When most experts are used anyway (many tokens), the dense products compute every expert for every
// token on the tensor cores and bfi_moe_weigh_dense multiplies the activations by the chosen experts'
// weights (0 for the others) between the two products:  act[t, e ff + j] *= weight of e for token t.
// An expert that every token uses may stand behind the routed ones in both matrices (`tail` more
// activations per token); its activations are multiplied by the token's gate.
#include "common.cuh"

__device__ __forceinline__ float moe_sigmoid(float x) {
    if (x >= 0.0f) return 1.0f / (1.0f + expf(-x));
    const float z = expf(x);
    return z / (1.0f + z);
}

// The decision of one token, by one warp: zr[0..E) are its logits (zr[E] the extra one), s, choice
// (E floats each) and gs (n_groups floats) are the warp's scratch in shared memory.
__device__ __forceinline__ void moe_route_token(const float* zr, const float* __restrict__ correction, int* __restrict__ idx,
                                                float* __restrict__ weight, float* __restrict__ gate, float* s, float* choice,
                                                float* gs, int t, int E, int top, int n_groups, int keep, float weight_scale,
                                                int extra, int lane, int score_mode, int group_top) {
    if (score_mode == 1) {
        for (int e = lane; e < E; e += 32) {
            s[e] = moe_sigmoid(zr[e]);
            choice[e] = s[e] + (correction ? correction[e] : 0.0f);
        }
    } else {
        float m = -INFINITY;
        for (int e = lane; e < E; e += 32) m = fmaxf(m, zr[e]);
        m = warp_max(m);
        float sum = 0.0f;
        for (int e = lane; e < E; e += 32) {
            const float p = expf(zr[e] - m);
            s[e] = p;
            sum += p;
        }
        sum = warp_sum(sum);
        const float inv = 1.0f / sum;
        for (int e = lane; e < E; e += 32) {
            s[e] *= inv;
            choice[e] = s[e] + (correction ? correction[e] : 0.0f);
        }
    }
    __syncwarp();
    const int per = E / n_groups;
    if (n_groups > 1 && keep < n_groups) {
        for (int g = lane; g < n_groups; g += 32) {
            float best = -INFINITY;
            if (group_top <= 1) {
                for (int e = g * per; e < (g + 1) * per; ++e) best = fmaxf(best, choice[e]);
            } else {
                // the sum of the group's `group_top` largest, picked one after the other; what an
                // earlier round picked is known by (value, position), so equal values count each
                best = 0.0f;
                int last_at = -1;
                float last_v = INFINITY;
                for (int r = 0; r < group_top && r < per; ++r) {
                    float bv = -INFINITY;
                    int ba = -1;
                    for (int e = g * per; e < (g + 1) * per; ++e) {
                        const float v = choice[e];
                        const bool open = v < last_v || (v == last_v && e > last_at);   // not picked in an earlier round
                        if (open && (v > bv || ba < 0)) bv = v, ba = e;
                    }
                    if (ba < 0) break;
                    best += bv;
                    last_v = bv, last_at = ba;
                }
            }
            gs[g] = best;
        }
        __syncwarp();
        // the `keep` best groups are marked by +inf in gs, one per round
        for (int r = 0; r < keep; ++r) {
            float best = -INFINITY;
            int at = 0x7fffffff;
            for (int g = lane; g < n_groups; g += 32) {
                const float v = gs[g];
                if (v != INFINITY && (v > best || (v == best && g < at))) best = v, at = g;
            }
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                if (ob > best || (ob == best && oa < at)) best = ob, at = oa;
            }
            if (lane == 0 && at != 0x7fffffff) gs[at] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (gs[e / per] != INFINITY) choice[e] = -INFINITY;
        __syncwarp();
    }
    for (int r = 0; r < top; ++r) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = choice[e];
            if (!isnan(v) && (v > best || (v == best && e < at))) best = v, at = e;
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) best = ob, at = oa;
        }
        if (at == 0x7fffffff) at = 0;                  // nothing left to choose from: expert 0 with weight 0
        if (lane == 0) {
            idx[(size_t)t * top + r] = at;
            weight[(size_t)t * top + r] = best == -INFINITY ? 0.0f : s[at] * weight_scale;
            choice[at] = NAN;                          // taken
        }
        __syncwarp();
    }
    if (extra && lane == 0) gate[t] = moe_sigmoid(zr[E]);
}

// One warp per token, logits given.  Shared memory per warp: s[E], choice[E], group[n_groups].
__global__ void moe_route_kernel(const float* __restrict__ z, long z_stride, const float* __restrict__ correction,
                                 int* __restrict__ idx, float* __restrict__ weight, float* __restrict__ gate,
                                 int n_tokens, int E, int top, int n_groups, int keep, float weight_scale, int extra,
                                 int score_mode, int group_top) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float sm[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int t = blockIdx.x * n_warps + warp;
    if (t >= n_tokens) return;
    float* s = sm + (size_t)warp * (2 * E + n_groups);
    moe_route_token(z + (size_t)t * z_stride, correction, idx, weight, gate, s, s + E, s + 2 * E, t, E, top, n_groups, keep,
                    weight_scale, extra, lane, score_mode, group_top);
}

extern "C" int bfi_moe_route(const float* z, long z_stride, const float* correction, int* idx, float* weight, float* gate,
                             int n_tokens, int E, int top, int n_groups, int keep, float weight_scale, int extra,
                             int score_mode, int group_top, cudaStream_t stream) {
    BFI_REQUIRE(E > 0 && top > 0 && top <= E, "moe_route: cannot choose %d of %d experts", top, E);
    BFI_REQUIRE((score_mode == 0 || score_mode == 1) && group_top >= 1, "moe_route: unknown score mode or group rule");
    BFI_REQUIRE(n_groups > 0 && E % n_groups == 0 && keep > 0 && keep <= n_groups,
                "moe_route: %d experts in %d groups, %d kept", E, n_groups, keep);
    BFI_REQUIRE((long)keep * (E / n_groups) >= top, "moe_route: %d groups of %d experts cannot give %d", keep, E / n_groups, top);
    BFI_REQUIRE(z_stride >= E + (extra ? 1 : 0), "moe_route: a row of logits is shorter than the experts");
    BFI_REQUIRE(!extra || gate != nullptr, "moe_route: the extra logit needs a place for its gate");
    if (n_tokens <= 0) return 0;
    const int warps = 4;
    const size_t smem = (size_t)warps * (2 * E + n_groups) * sizeof(float);
    BFI_REQUIRE(smem <= 48 * 1024, "moe_route: %d experts are too many for this kernel", E);
    bfi_launch(moe_route_kernel, dim3((n_tokens + warps - 1) / warps), dim3(32 * warps), smem, stream, z, z_stride, correction,
               idx, weight, gate, n_tokens, E, top, n_groups, keep, weight_scale, extra, score_mode, group_top);
    return bfi_check_launch("moe_route");
}

// dot of a weight row (storage T) with a float32 vector in shared memory, across a warp
template <typename T>
__device__ __forceinline__ float warp_dot(const T* __restrict__ w, const float* __restrict__ x, int n, int lane);

// (x is 16-byte aligned; the loops are unrolled so that several of a row's loads are in flight at once)
template <>
__device__ __forceinline__ float warp_dot<float>(const float* __restrict__ w, const float* __restrict__ x, int n, int lane) {
    float acc0 = 0.0f, acc1 = 0.0f;
    if ((n & 3) == 0 && ((uintptr_t)w & 15) == 0) {
#pragma unroll 4
        for (int j = lane * 4; j < n; j += 128) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(w + j));
            const float4 b = *reinterpret_cast<const float4*>(x + j);
            acc0 = fmaf(a.x, b.x, acc0), acc1 = fmaf(a.y, b.y, acc1), acc0 = fmaf(a.z, b.z, acc0), acc1 = fmaf(a.w, b.w, acc1);
        }
    } else {
#pragma unroll 4
        for (int j = lane; j < n; j += 32) acc0 = fmaf(w[j], x[j], acc0);
    }
    return warp_sum(acc0 + acc1);
}
template <>
__device__ __forceinline__ float warp_dot<bf16>(const bf16* __restrict__ w, const float* __restrict__ x, int n, int lane) {
    float acc0 = 0.0f, acc1 = 0.0f;
    if ((n & 7) == 0 && ((uintptr_t)w & 15) == 0) {
#pragma unroll 4
        for (int j = lane * 8; j < n; j += 256) {
            const uint4 raw = __ldg(reinterpret_cast<const uint4*>(w + j));
            const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
            const float4 b0 = *reinterpret_cast<const float4*>(x + j);
            const float4 b1 = *reinterpret_cast<const float4*>(x + j + 4);
            const float2 f0 = __bfloat1622float2(p[0]), f1 = __bfloat1622float2(p[1]);
            const float2 f2 = __bfloat1622float2(p[2]), f3 = __bfloat1622float2(p[3]);
            acc0 = fmaf(f0.x, b0.x, acc0), acc1 = fmaf(f0.y, b0.y, acc1), acc0 = fmaf(f1.x, b0.z, acc0), acc1 = fmaf(f1.y, b0.w, acc1);
            acc0 = fmaf(f2.x, b1.x, acc0), acc1 = fmaf(f2.y, b1.y, acc1), acc0 = fmaf(f3.x, b1.z, acc0), acc1 = fmaf(f3.y, b1.w, acc1);
        }
    } else {
#pragma unroll 4
        for (int j = lane; j < n; j += 32) acc0 = fmaf(__bfloat162float(w[j]), x[j], acc0);
    }
    return warp_sum(acc0 + acc1);
}

// The router's logits and its decision in one kernel: one block per token, the token's input as
// float32 in shared memory, a warp per logit (router rows are float32 [E (+1), width]), then warp 0
// decides.  The logits are float32 sums of float32 products of the input as its storage type holds it.
template <typename T>
__global__ void __launch_bounds__(256)
moe_router_kernel(const T* __restrict__ h, long h_stride, const float* __restrict__ w_router,
                  const float* __restrict__ correction, const int* __restrict__ token_slot, int* __restrict__ idx,
                  float* __restrict__ weight, float* __restrict__ gate, int width, int E, int top, int n_groups, int keep,
                  float weight_scale, int extra, int score_mode, int group_top) {
    pdl_trigger();
    extern __shared__ __align__(16) float sm[];
    float* hs = sm;                                // [width]
    float* z = hs + width;                         // [E + 1]
    float* scratch = z + E + 1;                    // [2 E + n_groups]
    const int t = blockIdx.x;
    if (token_slot[t] < 0) return;
    pdl_wait();
    for (int j = threadIdx.x; j < width; j += blockDim.x) hs[j] = to_f32(h[(size_t)t * h_stride + j]);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    for (int e = warp; e < E + (extra ? 1 : 0); e += n_warps) {
        const float d = warp_dot<float>(w_router + (size_t)e * width, hs, width, lane);
        if (lane == 0) z[e] = d;
    }
    __syncthreads();
    if (warp == 0)
        moe_route_token(z, correction, idx, weight, gate, scratch, scratch + E, scratch + 2 * E, t, E, top, n_groups, keep,
                        weight_scale, extra, lane, score_mode, group_top);
}

extern "C" int bfi_moe_router(const void* h, long h_stride, int dtype, const float* w_router, const float* correction,
                              const int* token_slot, int* idx, float* weight, float* gate, int n_tokens, int width, int E,
                              int top, int n_groups, int keep, float weight_scale, int extra, int score_mode, int group_top,
                              cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(dtype), "moe_router: unknown dtype code %d", dtype);
    BFI_REQUIRE((score_mode == 0 || score_mode == 1) && group_top >= 1, "moe_router: unknown score mode or group rule");
    BFI_REQUIRE(E > 0 && top > 0 && top <= E && width > 0 && h_stride >= width, "moe_router: cannot choose %d of %d experts", top, E);
    BFI_REQUIRE(n_groups > 0 && E % n_groups == 0 && keep > 0 && keep <= n_groups,
                "moe_router: %d experts in %d groups, %d kept", E, n_groups, keep);
    BFI_REQUIRE((long)keep * (E / n_groups) >= top, "moe_router: %d groups of %d experts cannot give %d", keep, E / n_groups, top);
    BFI_REQUIRE(!extra || gate != nullptr, "moe_router: the extra logit needs a place for its gate");
    if (n_tokens <= 0) return 0;
    const size_t smem = (size_t)(width + 3 * E + 1 + n_groups) * sizeof(float);
    BFI_REQUIRE(smem <= 160 * 1024, "moe_router: width %d and %d experts do not fit shared memory", width, E);
    cudaError_t e = cudaSuccess;
    if (dtype == BFI_F32) {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(moe_router_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess)
            bfi_launch(moe_router_kernel<float>, dim3(n_tokens), dim3(256), smem, stream, (const float*)h, h_stride, w_router, correction,
                       token_slot, idx, weight, gate, width, E, top, n_groups, keep, weight_scale, extra, score_mode, group_top);
    } else {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(moe_router_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess)
            bfi_launch(moe_router_kernel<bf16>, dim3(n_tokens), dim3(256), smem, stream, (const bf16*)h, h_stride, w_router, correction,
                       token_slot, idx, weight, gate, width, E, top, n_groups, keep, weight_scale, extra, score_mode, group_top);
    }
    if (e != cudaSuccess) return bfi_fail("moe_router: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    return bfi_check_launch("moe_router");
}

#define MOE_WARPS 8

// grid (pairs, chunks of ff rows)
template <typename T>
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_gate_up_kernel(const T* __restrict__ h, long h_stride, const T* __restrict__ w_gu,
                   const int* __restrict__ idx, const int* __restrict__ token_slot, T* __restrict__ act, int top,
                   int width, int ff, int rows_per_block, int act_kind) {
    pdl_trigger();
    extern __shared__ __align__(16) float hs[];    // [width]
    const int pair = blockIdx.x;
    const int t = pair / top;
    if (token_slot[t] < 0) return;                 // padding row
    pdl_wait();
    const int e = idx != nullptr ? idx[pair] : 0;          // no choices: one expert that every token uses
    for (int j = threadIdx.x; j < width; j += blockDim.x) hs[j] = to_f32(h[(size_t)t * h_stride + j]);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r0 = blockIdx.y * rows_per_block;
    const int r1 = min(ff, r0 + rows_per_block);
    if (act_kind == 1) {
        for (int r = r0 + warp; r < r1; r += MOE_WARPS) {
            const float u = fmaxf(warp_dot<T>(w_gu + ((size_t)e * ff + r) * width, hs, width, lane), 0.0f);
            if (lane == 0) act[(size_t)pair * ff + r] = from_f32<T>(u * u);
        }
        return;
    }
    for (int r = r0 + warp; r < r1; r += MOE_WARPS) {
        const size_t off = ((size_t)e * ff + r) * 2 * width;
        const float g = warp_dot<T>(w_gu + off, hs, width, lane);
        const float u = warp_dot<T>(w_gu + off + width, hs, width, lane);
        if (lane == 0) act[(size_t)pair * ff + r] = from_f32<T>(g * moe_sigmoid(g) * u);
    }
}

extern "C" int bfi_moe_gate_up(const void* h, long h_stride, int dtype, const void* w_gu,
                               const int* idx, const int* token_slot, void* act, int n_tokens, int top, int width, int ff,
                               int act_kind, cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(dtype), "moe_gate_up: unknown dtype code %d", dtype);
    BFI_REQUIRE(act_kind == 0 || act_kind == 1, "moe_gate_up: unknown activation kind %d", act_kind);
    BFI_REQUIRE(top > 0 && width > 0 && ff > 0 && h_stride >= width, "moe_gate_up: bad sizes");
    if (n_tokens <= 0) return 0;
    const long pairs = (long)n_tokens * top;
    BFI_REQUIRE(pairs <= 2147483647L, "moe_gate_up: too many (token, expert) pairs");
    BFI_REQUIRE((size_t)width * 4 <= 160 * 1024, "moe_gate_up: a row of %d values does not fit shared memory", width);
    // enough blocks to fill the device when pairs are few, whole experts per block when they are many
    int chunks = 1;
    const int sms = bfi_sm_count();
    while (pairs * chunks < 4L * sms && chunks * MOE_WARPS < ff) chunks *= 2;
    const int rows_per_block = (ff + chunks - 1) / chunks;
    chunks = (ff + rows_per_block - 1) / rows_per_block;
    const size_t smem = (size_t)width * sizeof(float);
    const dim3 grid((unsigned)pairs, chunks);
    cudaError_t e = cudaSuccess;
    if (dtype == BFI_F32) {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(moe_gate_up_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess)
            bfi_launch(moe_gate_up_kernel<float>, grid, dim3(MOE_WARPS * 32), smem, stream, (const float*)h, h_stride,
                       (const float*)w_gu, idx, token_slot, (float*)act, top, width, ff, rows_per_block, act_kind);
    } else {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(moe_gate_up_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess)
            bfi_launch(moe_gate_up_kernel<bf16>, grid, dim3(MOE_WARPS * 32), smem, stream, (const bf16*)h, h_stride,
                       (const bf16*)w_gu, idx, token_slot, (bf16*)act, top, width, ff, rows_per_block, act_kind);
    }
    if (e != cudaSuccess) return bfi_fail("moe_gate_up: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    return bfi_check_launch("moe_gate_up");
}

// grid (tokens, chunks of output columns)
template <typename T>
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_down_kernel(const T* __restrict__ act, const T* __restrict__ w_down, const int* __restrict__ idx,
                const float* __restrict__ weight, const int* __restrict__ token_slot, const float* __restrict__ shared_out,
                long shared_stride, const float* __restrict__ gate, float* __restrict__ out, long out_stride, int top,
                int width, int ff, long ld, int cols_per_block, int accumulate) {
    pdl_trigger();
    extern __shared__ __align__(16) float as[];    // [top][ff]
    const int t = blockIdx.x;
    if (token_slot[t] < 0) return;
    pdl_wait();
    for (int j = threadIdx.x; j < top * ff; j += blockDim.x) as[j] = to_f32(act[(size_t)t * top * ff + j]);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int c0 = blockIdx.y * cols_per_block;
    const int c1 = min(width, c0 + cols_per_block);
    const float g = gate ? gate[t] : 1.0f;
    for (int c = c0 + warp; c < c1; c += MOE_WARPS) {
        float sum = 0.0f;
        for (int k = 0; k < top; ++k) {
            const int e = idx[(size_t)t * top + k];
            const float d = warp_dot<T>(w_down + (size_t)c * ld + (size_t)e * ff, as + (size_t)k * ff, ff, lane);
            sum = fmaf(weight[(size_t)t * top + k], d, sum);
        }
        if (lane == 0) {
            if (shared_out) sum = fmaf(g, shared_out[(size_t)t * shared_stride + c], sum);
            float* o = out + (size_t)t * out_stride + c;
            *o = accumulate ? *o + sum : sum;
        }
    }
}

extern "C" int bfi_moe_down(const void* act, int dtype, const void* w_down, const int* idx, const float* weight,
                            const int* token_slot, const float* shared_out, long shared_stride, const float* gate,
                            float* out, long out_stride, int n_tokens, int top, int width, int ff, long ld,
                            int accumulate, cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(dtype), "moe_down: unknown dtype code %d", dtype);
    BFI_REQUIRE(top > 0 && width > 0 && ff > 0 && out_stride >= width, "moe_down: bad sizes");
    BFI_REQUIRE(!shared_out || shared_stride >= width, "moe_down: the shared output's rows are shorter than the width");
    if (n_tokens <= 0) return 0;
    const size_t smem = (size_t)top * ff * sizeof(float);
    BFI_REQUIRE(smem <= 160 * 1024, "moe_down: %d x %d activations per token do not fit shared memory", top, ff);
    int chunks = 1;
    const int sms = bfi_sm_count();
    while ((long)n_tokens * chunks < 4L * sms && chunks * MOE_WARPS < width) chunks *= 2;
    const int cols_per_block = (width + chunks - 1) / chunks;
    chunks = (width + cols_per_block - 1) / cols_per_block;
    const dim3 grid(n_tokens, chunks);
    cudaError_t e = cudaSuccess;
    if (dtype == BFI_F32) {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(moe_down_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess)
            bfi_launch(moe_down_kernel<float>, grid, dim3(MOE_WARPS * 32), smem, stream, (const float*)act, (const float*)w_down, idx,
                       weight, token_slot, shared_out, shared_stride, gate, out, out_stride, top, width, ff, ld, cols_per_block,
                       accumulate);
    } else {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(moe_down_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess)
            bfi_launch(moe_down_kernel<bf16>, grid, dim3(MOE_WARPS * 32), smem, stream, (const bf16*)act, (const bf16*)w_down, idx,
                       weight, token_slot, shared_out, shared_stride, gate, out, out_stride, top, width, ff, ld, cols_per_block,
                       accumulate);
    }
    if (e != cudaSuccess) return bfi_fail("moe_down: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    return bfi_check_launch("moe_down");
}

// one block per token; act [tokens][E * ff + tail]
template <typename T>
__global__ void moe_weigh_dense_kernel(T* __restrict__ act, long act_stride, const int* __restrict__ idx,
                                       const float* __restrict__ weight, const int* __restrict__ token_slot, int top, int E,
                                       int ff, int tail, const float* __restrict__ gate, int act_kind) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float comb[];                // [E] the token's weight of every expert
    const int t = blockIdx.x;
    if (token_slot[t] < 0) return;
    for (int e = threadIdx.x; e < E; e += blockDim.x) comb[e] = 0.0f;
    __syncthreads();
    if (threadIdx.x < top) comb[idx[(size_t)t * top + threadIdx.x]] = weight[(size_t)t * top + threadIdx.x];
    __syncthreads();
    T* row = act + (size_t)t * act_stride;
    if (act_kind == 1) {
        // the row holds the up products themselves: relu(u)^2, rounded as the other way of computing
        // rounds it, then the weight
        for (int j = threadIdx.x; j < E * ff; j += blockDim.x) {
            const float c = comb[j / ff];
            const float u = fmaxf(to_f32(row[j]), 0.0f);
            row[j] = c == 0.0f ? from_f32<T>(0.0f) : from_f32<T>(to_f32(from_f32<T>(u * u)) * c);
        }
        const float g = gate != nullptr ? gate[t] : 1.0f;
        for (int j = E * ff + threadIdx.x; j < E * ff + tail; j += blockDim.x) {
            const float u = fmaxf(to_f32(row[j]), 0.0f);
            row[j] = gate != nullptr ? from_f32<T>(to_f32(from_f32<T>(u * u)) * g) : from_f32<T>(u * u);
        }
        return;
    }
    for (int j = threadIdx.x; j < E * ff; j += blockDim.x) {
        const float c = comb[j / ff];
        row[j] = c == 0.0f ? from_f32<T>(0.0f) : from_f32<T>(to_f32(row[j]) * c);
    }
    if (tail > 0 && gate != nullptr) {
        const float g = gate[t];
        for (int j = E * ff + threadIdx.x; j < E * ff + tail; j += blockDim.x) row[j] = from_f32<T>(to_f32(row[j]) * g);
    }
}

extern "C" int bfi_moe_weigh_dense(void* act, long act_stride, int dtype, const int* idx, const float* weight,
                                   const int* token_slot, int n_tokens, int top, int E, int ff, int tail, const float* gate,
                                   int act_kind, cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(dtype), "moe_weigh_dense: unknown dtype code %d", dtype);
    BFI_REQUIRE(act_kind == 0 || act_kind == 1, "moe_weigh_dense: unknown activation kind %d", act_kind);
    BFI_REQUIRE(top > 0 && top <= 1024 && E > 0 && ff > 0 && tail >= 0 && act_stride >= (long)E * ff + tail,
                "moe_weigh_dense: bad sizes");
    if (n_tokens <= 0) return 0;
    const size_t smem = (size_t)E * sizeof(float);
    BFI_REQUIRE(smem <= 48 * 1024, "moe_weigh_dense: %d experts are too many for this kernel", E);
    const int threads = top > 256 ? 1024 : 256;
    if (dtype == BFI_F32)
        bfi_launch(moe_weigh_dense_kernel<float>, dim3(n_tokens), dim3(threads), smem, stream, (float*)act, act_stride, idx, weight,
                   token_slot, top, E, ff, tail, gate, act_kind);
    else
        bfi_launch(moe_weigh_dense_kernel<bf16>, dim3(n_tokens), dim3(threads), smem, stream, (bf16*)act, act_stride, idx, weight,
                   token_slot, top, E, ff, tail, gate, act_kind);
    return bfi_check_launch("moe_weigh_dense");
}

BFI_TRACE_EXPORT(moe)
