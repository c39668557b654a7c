// Linear recurrences with a decay that depends on the token, and what stands around them: the
// general kernels (any sizes, any step shape: whole prompts, further pieces, single tokens),
// float32 or bfloat16 storage of the inputs, float32 arithmetic and float32 state.
//
// Per sequence and head, with q_t, k_t (D values) and v_t (V values):
//     S_t = diag(a_t) S_(t-1) + k_t (c_t v_t)^T          S is D x V, float32, kept per slot
//     o_t = S_t^T q_t + skip * v_t
// The decay a_t and the factor c_t come from a raw value r of the token (a projection's output)
// in one of these forms, all evaluated here in float32:
//     REC_DECAY_STEP      one r per head:   c = softplus(r + bias_h), a = exp(-rate_h * c) for all rows
//                         (a discretised state space: c is the step size, rate_h > 0)
//     REC_DECAY_SIGMOID   one r per row d:  a_d = sigmoid(r + bias_(h,d))^(1/tau), c = 1
// Heads may share q and k in groups (q_t and k_t of head h are those of group h / heads_per_group).
// Column j of S, and with it value j of o, depends on no other column, so a block owns a range of
// columns of one head of one sequence and walks the sequence's new tokens in order.
//
// bfi_causal_conv: a short causal convolution per channel over the step's tokens (with silu or
// without), whose last taps-1 inputs per sequence are kept as state (zero before the first token).
// bfi_gated_group_norm: the gate and the norm in equal parts that follow such a recurrence.
#include "common.cuh"

#define REC_DECAY_STEP 1
#define REC_DECAY_SIGMOID 2
#define REC_MAX_TAPS 16

__device__ __forceinline__ float rec_sigmoid(float x) {
    if (x >= 0.0f) return 1.0f / (1.0f + expf(-x));
    const float z = expf(x);
    return z / (1.0f + z);
}
__device__ __forceinline__ float rec_silu(float x) { return x * rec_sigmoid(x); }
__device__ __forceinline__ float rec_softplus(float x) { return fmaxf(x, 0.0f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float rec_log_sigmoid(float x) { return fminf(x, 0.0f) - log1pf(expf(-fabsf(x))); }

struct RecArgs {
    long qk_stride, v_stride, r_stride, out_stride;   // elements between tokens
    int q_off, k_off, v_off, r_off;                    // first column of each in its row
    int H, D, V, heads_per_group;
    int mode;
    float q_scale, inv_tau;
    const float *bias, *rate, *skip;                   // float32: [H] or [H*D] bias, [H] rate, [H] skip (or null)
    const int *cu_seqlens, *seq_slot;
    int vb, v_blocks, chunk_len;
};

// PHASE 0: a sequence's new tokens in order, from the slot's state, which is moved on.
// The other phases cut every sequence into chunks of `chunk_len` tokens that run side by side
// (blockIdx.z is the chunk; chunk c of sequence s has the running number base(s) + c, where base
// counts the chunks of the sequences before s):
// PHASE 1: a chunk alone from a zero state: out gets the part of o that the chunk's own tokens give,
//          chunk_state[n] the state the chunk adds (sum_j diag(prod_{i>j} a_i) k_j (c_j v_j)^T) and
//          chunk_decay[n] the product of the chunk's decays per row.
// (between them decay_chunk_carry_kernel walks the chunks of a sequence in order and leaves in
//  chunk_state[n] the state that chunk n starts from, and in the slot's state the one after the last)
// PHASE 3: out += (q_t * prod_{i<=t in chunk} a_i)^T chunk_state[n]: what the tokens before the chunk give.
template <typename T, int PHASE>
__global__ void decay_scan_kernel(const T* __restrict__ qk, const T* __restrict__ vsrc, const T* __restrict__ raw,
                                  float* __restrict__ out, float* __restrict__ state, float* __restrict__ chunk_state,
                                  float* __restrict__ chunk_decay, const RecArgs a) {
    pdl_trigger();
    extern __shared__ float sm[];
    const int D = a.D, V = a.V, vb = a.vb;
    float* S = sm;                      // [D][vb]
    float* qs = S + (size_t)D * vb;     // [D]
    float* ks = qs + D;                 // [D]
    float* as = ks + D;                 // [D] decay per row
    float* ps = as + D;                 // [D] product of the chunk's decays so far per row
    float* red = ps + D;                // [threads]
    __shared__ float step_c;
    const int seq = blockIdx.y;
    const int slot = a.seq_slot[seq];
    if (slot < 0) return;
    const int h = blockIdx.x / a.v_blocks;
    const int v0 = (blockIdx.x - h * a.v_blocks) * vb;
    int t0 = a.cu_seqlens[seq], nt = a.cu_seqlens[seq + 1] - t0;
    size_t chunk_no = 0;
    if (PHASE != 0) {
        const int first = blockIdx.z * a.chunk_len;
        if (first >= nt) return;
        for (int s2 = 0; s2 < seq; ++s2)
            chunk_no += (a.cu_seqlens[s2 + 1] - a.cu_seqlens[s2] + a.chunk_len - 1) / a.chunk_len;
        chunk_no += blockIdx.z;
        t0 += first;
        nt = min(a.chunk_len, nt - first);
    }
    const int c = threadIdx.x % vb, g = threadIdx.x / vb, ng = blockDim.x / vb;
    const bool col_ok = v0 + c < V;
    const int grp = h / a.heads_per_group;
    const float skip = a.skip ? a.skip[h] : 0.0f;
    // the state of earlier steps (zeroed when the slot was taken) does not come from this step's kernels
    float* sp = PHASE == 0 ? state + (((size_t)slot * a.H + h) * D) * V + v0
                           : chunk_state + ((chunk_no * a.H + h) * D) * V + v0;
    if (PHASE == 0) {
        for (int d = g; d < D; d += ng) S[d * vb + c] = col_ok ? sp[(size_t)d * V + c] : 0.0f;
        pdl_wait();
    } else {
        pdl_wait();
        for (int d = g; d < D; d += ng) S[d * vb + c] = (PHASE == 3 && col_ok) ? sp[(size_t)d * V + c] : 0.0f;
        for (int j = threadIdx.x; j < D; j += blockDim.x) ps[j] = 1.0f;
    }
    for (int t = 0; t < nt; ++t) {
        const size_t tok = (size_t)(t0 + t);
        const T* row = qk + tok * a.qk_stride + (size_t)grp * D;
        const T* rr = raw + tok * a.r_stride + a.r_off;
        if (a.mode == REC_DECAY_STEP) {
            if (threadIdx.x == 0) step_c = rec_softplus(to_f32(rr[h]) + a.bias[h]);
            __syncthreads();
            const float w = expf(-a.rate[h] * step_c);
            for (int j = threadIdx.x; j < D; j += blockDim.x) {
                qs[j] = to_f32(row[a.q_off + j]) * a.q_scale;
                if (PHASE != 3) ks[j] = to_f32(row[a.k_off + j]);
                as[j] = w;
                if (PHASE != 0) ps[j] *= w;
            }
        } else {
            if (threadIdx.x == 0) step_c = 1.0f;
            for (int j = threadIdx.x; j < D; j += blockDim.x) {
                qs[j] = to_f32(row[a.q_off + j]) * a.q_scale;
                if (PHASE != 3) ks[j] = to_f32(row[a.k_off + j]);
                const float w = expf(rec_log_sigmoid(to_f32(rr[(size_t)h * D + j]) + a.bias[(size_t)h * D + j]) * a.inv_tau);
                as[j] = w;
                if (PHASE != 0) ps[j] *= w;
            }
        }
        float vv = 0.0f;
        if (PHASE != 3 && col_ok) vv = to_f32(vsrc[tok * a.v_stride + a.v_off + (size_t)h * V + v0 + c]);
        __syncthreads();
        float acc = 0.0f;
        if (PHASE == 3) {
            for (int d = g; d < D; d += ng) acc = fmaf(S[d * vb + c], qs[d] * ps[d], acc);
        } else {
            const float cv = step_c * vv;
            for (int d = g; d < D; d += ng) {
                const float s = fmaf(as[d], S[d * vb + c], ks[d] * cv);
                S[d * vb + c] = s;
                acc = fmaf(s, qs[d], acc);
            }
        }
        red[threadIdx.x] = acc;
        __syncthreads();
        if (threadIdx.x < vb && col_ok) {
            float o = 0.0f;
            for (int i = 0; i < ng; ++i) o += red[i * vb + threadIdx.x];
            float* dst = out + tok * a.out_stride + (size_t)h * V + v0 + c;
            if (PHASE == 3) *dst += o;
            else *dst = fmaf(skip, vv, o);
        }
    }
    if (PHASE != 3 && col_ok)
        for (int d = g; d < D; d += ng) sp[(size_t)d * V + c] = S[d * vb + c];
    if (PHASE == 1 && v0 == 0)
        for (int j = threadIdx.x; j < D; j += blockDim.x) chunk_decay[(chunk_no * a.H + h) * D + j] = ps[j];
}

// The same three phases with the state in registers, for D up to 128: a block of four warps owns up to
// 128 columns of one head of one sequence (or chunk), a warp 32 of them, and lane l of a warp holds all
// D rows of its column, so a token's output value is one thread's sum (four partial sums).  The block
// shares the work on a token's q, k and decay: thread i fetches row i (one token ahead of the
// arithmetic, kept in its storage type until used), evaluates the row's decay and puts the three values
// into one of two buffers in shared memory, which all warps then read; with two buffers one barrier a
// token is enough (whoever writes token t + 1 has passed the barrier of token t, which nobody reaches
// before it has finished reading token t - 1).
#define REC_WARPS 4

template <typename T, int PHASE, int MODE, int DMAX>
__global__ void __launch_bounds__(REC_WARPS * 32)
decay_scan_regs_kernel(const T* __restrict__ qk, const T* __restrict__ vsrc, const T* __restrict__ raw,
                       float* __restrict__ out, float* __restrict__ state, float* __restrict__ chunk_state,
                       float* __restrict__ chunk_decay, const RecArgs a) {
    pdl_trigger();
    __shared__ __align__(16) float stage[2][3][DMAX];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, tid = threadIdx.x;
    const int seq = blockIdx.y;
    const int slot = a.seq_slot[seq];
    if (slot < 0) return;
    const int D = a.D, V = a.V;
    const int h = blockIdx.x / a.v_blocks;                      // v_blocks: groups of 128 columns
    const int col = (blockIdx.x - h * a.v_blocks) * (REC_WARPS * 32) + warp * 32 + lane;
    const bool col_ok = col < V;
    const bool warp_ok = col - lane < V;                        // the warp has a column at all
    int t0 = a.cu_seqlens[seq], nt = a.cu_seqlens[seq + 1] - t0;
    size_t chunk_no = 0;
    if (PHASE != 0) {
        const int first = blockIdx.z * a.chunk_len;
        if (first >= nt) return;
        for (int s2 = 0; s2 < seq; ++s2)
            chunk_no += (a.cu_seqlens[s2 + 1] - a.cu_seqlens[s2] + a.chunk_len - 1) / a.chunk_len;
        chunk_no += blockIdx.z;
        t0 += first;
        nt = min(a.chunk_len, nt - first);
    }
    const int grp = h / a.heads_per_group;
    const float skip = a.skip ? a.skip[h] : 0.0f;
    float* sp = PHASE == 0 ? state + (((size_t)slot * a.H + h) * D) * V + col
                           : chunk_state + ((chunk_no * a.H + h) * D) * V + col;
    float S[DMAX];
    if (PHASE == 0) {
#pragma unroll
        for (int d = 0; d < DMAX; ++d) S[d] = (col_ok && d < D) ? sp[(size_t)d * V] : 0.0f;
        pdl_wait();
    } else {
        pdl_wait();
#pragma unroll
        for (int d = 0; d < DMAX; ++d) S[d] = (PHASE == 3 && col_ok && d < D) ? sp[(size_t)d * V] : 0.0f;
    }
    // this thread's row (threads past DMAX have none), its decay's constant and the running product
    // of the chunk's decays
    const bool row_mine = tid < DMAX, row_ok = tid < D;
    const float bias_r = (MODE == REC_DECAY_SIGMOID && row_ok) ? a.bias[(size_t)h * D + tid] : 0.0f;
    const float bias_h = MODE == REC_DECAY_STEP ? a.bias[h] : 0.0f;
    const float rate_h = MODE == REC_DECAY_STEP ? a.rate[h] : 0.0f;
    float prod = 1.0f;
    T nq = from_f32<T>(0.0f), nk = nq, nr = nq, nv = nq, nstep = nq;
    float nold = 0.0f;
    auto fetch = [&](int t) {
        const size_t tok = (size_t)(t0 + t);
        const T* row = qk + tok * a.qk_stride + (size_t)grp * D;
        const T* rr = raw + tok * a.r_stride + a.r_off;
        if (row_ok) {
            nq = row[a.q_off + tid];
            if (PHASE != 3) nk = row[a.k_off + tid];
            if (MODE == REC_DECAY_SIGMOID) nr = rr[(size_t)h * D + tid];
        }
        if (MODE == REC_DECAY_STEP) nstep = rr[h];
        if (PHASE != 3 && col_ok) nv = vsrc[tok * a.v_stride + a.v_off + (size_t)h * V + col];
        if (PHASE == 3 && col_ok) nold = out[tok * a.out_stride + (size_t)h * V + col];
    };
    if (nt > 0) fetch(0);
    for (int t = 0; t < nt; ++t) {
        float* qs = stage[t & 1][0];
        float* ks = stage[t & 1][1];
        float* as = stage[t & 1][2];
        float step_c = 1.0f, w_h = 1.0f;
        if (MODE == REC_DECAY_STEP) {
            step_c = rec_softplus(to_f32(nstep) + bias_h);
            w_h = expf(-rate_h * step_c);
        }
        if (row_mine) {
            float w = MODE == REC_DECAY_STEP ? w_h : expf(rec_log_sigmoid(to_f32(nr) + bias_r) * a.inv_tau);
            if (!row_ok) w = 1.0f;
            if (PHASE != 0) prod *= w;
            qs[tid] = row_ok ? to_f32(nq) * a.q_scale * (PHASE == 3 ? prod : 1.0f) : 0.0f;
            if (PHASE != 3) ks[tid] = row_ok ? to_f32(nk) : 0.0f;
            if (MODE == REC_DECAY_SIGMOID && PHASE != 3) as[tid] = w;
        }
        const float old = nold;
        const float vv = to_f32(nv);
        __syncthreads();
        if (t + 1 < nt) fetch(t + 1);
        if (!warp_ok) continue;
        const float cv = step_c * vv;
        // four partial sums, so that a token's sum is four chains of D / 4 dependent operations
        float acc0 = 0.0f, acc1 = 0.0f, acc2 = 0.0f, acc3 = 0.0f;
        // rows past D hold q = k = 0, a = 1 and a zero state, so whole groups of 16 rows are walked
        // and only groups that start past D are skipped
#pragma unroll
        for (int d16 = 0; d16 < DMAX; d16 += 16) {
            if (d16 < D) {
#pragma unroll
                for (int d4 = d16; d4 < d16 + 16; d4 += 4) {
                    const float4 q4 = *reinterpret_cast<const float4*>(qs + d4);
                    if (PHASE == 3) {
                        acc0 = fmaf(S[d4], q4.x, acc0), acc1 = fmaf(S[d4 + 1], q4.y, acc1);
                        acc2 = fmaf(S[d4 + 2], q4.z, acc2), acc3 = fmaf(S[d4 + 3], q4.w, acc3);
                    } else {
                        const float4 k4 = *reinterpret_cast<const float4*>(ks + d4);
                        float4 a4;
                        if (MODE == REC_DECAY_STEP) a4 = make_float4(w_h, w_h, w_h, w_h);
                        else a4 = *reinterpret_cast<const float4*>(as + d4);
                        S[d4] = fmaf(a4.x, S[d4], k4.x * cv), acc0 = fmaf(S[d4], q4.x, acc0);
                        S[d4 + 1] = fmaf(a4.y, S[d4 + 1], k4.y * cv), acc1 = fmaf(S[d4 + 1], q4.y, acc1);
                        S[d4 + 2] = fmaf(a4.z, S[d4 + 2], k4.z * cv), acc2 = fmaf(S[d4 + 2], q4.z, acc2);
                        S[d4 + 3] = fmaf(a4.w, S[d4 + 3], k4.w * cv), acc3 = fmaf(S[d4 + 3], q4.w, acc3);
                    }
                }
            }
        }
        const float acc = (acc0 + acc1) + (acc2 + acc3);
        if (col_ok) {
            float* dst = out + (size_t)(t0 + t) * a.out_stride + (size_t)h * V + col;
            if (PHASE == 3) *dst = old + acc;
            else *dst = fmaf(skip, vv, acc);
        }
    }
    if (PHASE != 3 && col_ok) {
#pragma unroll
        for (int d = 0; d < DMAX; ++d)
            if (d < D) sp[(size_t)d * V] = S[d];
    }
    if (PHASE == 1 && blockIdx.x == h * a.v_blocks && row_ok) chunk_decay[(chunk_no * a.H + h) * D + tid] = prod;
}

// One new token per sequence: the state never rests anywhere.  A warp owns 32 columns of one head of
// one sequence and streams the rows of its columns through once: read, decay, add, multiply by q, write.
// The rows are asked for sixteen at a time so that a step's traffic, which is the states read and
// written once, streams.
#define REC_STEP_DMAX 512
template <typename T, int MODE>
__global__ void __launch_bounds__(REC_WARPS * 32)
decay_step_kernel(const T* __restrict__ qk, const T* __restrict__ vsrc, const T* __restrict__ raw, float* __restrict__ out,
                  float* __restrict__ state, const RecArgs a) {
    pdl_trigger();
    extern __shared__ __align__(16) float step_stage[];          // [REC_WARPS][3][D rounded up to 4]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int unit = blockIdx.x * REC_WARPS + warp;
    const int seq = blockIdx.y;
    const int slot = a.seq_slot[seq];
    if (slot < 0 || unit >= a.H * a.v_blocks) return;
    const int D = a.D, V = a.V, Dp = (D + 3) & ~3;
    const int h = unit / a.v_blocks;
    const int col = (unit - h * a.v_blocks) * 32 + lane;
    const bool col_ok = col < V;
    const int grp = h / a.heads_per_group;
    float* qs = step_stage + (size_t)warp * 3 * Dp;
    float* ks = qs + Dp;
    float* as = ks + Dp;
    float* sp = state + (((size_t)slot * a.H + h) * D) * V + col;
    pdl_wait();
    const size_t tok = (size_t)a.cu_seqlens[seq];
    const T* row = qk + tok * a.qk_stride + (size_t)grp * D;
    const T* rr = raw + tok * a.r_stride + a.r_off;
    float step_c = 1.0f, w_h = 1.0f;
    if (MODE == REC_DECAY_STEP) {
        step_c = rec_softplus(to_f32(rr[h]) + a.bias[h]);
        w_h = expf(-a.rate[h] * step_c);
    }
    for (int d = lane; d < Dp; d += 32) {
        const bool in = d < D;
        qs[d] = in ? to_f32(row[a.q_off + d]) * a.q_scale : 0.0f;
        ks[d] = in ? to_f32(row[a.k_off + d]) : 0.0f;
        as[d] = !in ? 1.0f : (MODE == REC_DECAY_STEP ? w_h
                               : expf(rec_log_sigmoid(to_f32(rr[(size_t)h * D + d]) + a.bias[(size_t)h * D + d]) * a.inv_tau));
    }
    const float vv = col_ok ? to_f32(vsrc[tok * a.v_stride + a.v_off + (size_t)h * V + col]) : 0.0f;
    __syncwarp();
    if (!col_ok) return;
    const float cv = step_c * vv;
    float acc0 = 0.0f, acc1 = 0.0f;
    int d = 0;
    for (; d + 16 <= D; d += 16) {
        float sv[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) sv[i] = sp[(size_t)(d + i) * V];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            sv[i] = fmaf(as[d + i], sv[i], ks[d + i] * cv);
            sp[(size_t)(d + i) * V] = sv[i];
            if (i & 1) acc1 = fmaf(sv[i], qs[d + i], acc1);
            else acc0 = fmaf(sv[i], qs[d + i], acc0);
        }
    }
    for (; d < D; ++d) {
        const float s1 = fmaf(as[d], sp[(size_t)d * V], ks[d] * cv);
        sp[(size_t)d * V] = s1;
        acc0 = fmaf(s1, qs[d], acc0);
    }
    out[tok * a.out_stride + (size_t)h * V + col] = fmaf(a.skip ? a.skip[h] : 0.0f, vv, acc0 + acc1);
}

template <typename T>
static int launch_decay_step(const void* qk, const void* vsrc, const void* raw, float* out, float* state, RecArgs a, int n_seqs,
                             cudaStream_t stream) {
    a.vb = 32, a.v_blocks = (a.V + 31) / 32;
    const dim3 grid((a.H * a.v_blocks + REC_WARPS - 1) / REC_WARPS, n_seqs), block(REC_WARPS * 32);
    const size_t smem = (size_t)REC_WARPS * 3 * ((a.D + 3) & ~3) * sizeof(float);
    if (a.mode == REC_DECAY_STEP)
        bfi_launch(decay_step_kernel<T, REC_DECAY_STEP>, grid, block, smem, stream, (const T*)qk, (const T*)vsrc, (const T*)raw, out,
                   state, a);
    else
        bfi_launch(decay_step_kernel<T, REC_DECAY_SIGMOID>, grid, block, smem, stream, (const T*)qk, (const T*)vsrc, (const T*)raw,
                   out, state, a);
    return bfi_check_launch("decay_scan (single tokens)");
}

// One thread per element of a head's state: S = state[slot]; for every chunk of the sequence in
// order: the chunk's place receives S (the state it starts from) and S = decay_row * S + what the
// chunk adds; at the end state[slot] = S.
__global__ void decay_chunk_carry_kernel(float* __restrict__ state, float* __restrict__ chunk_state,
                                         const float* __restrict__ chunk_decay, const int* __restrict__ cu_seqlens,
                                         const int* __restrict__ seq_slot, int H, int D, int V, int chunk_len) {
    pdl_trigger();
    pdl_wait();
    const int seq = blockIdx.z, h = blockIdx.y;
    const int slot = seq_slot[seq];
    if (slot < 0) return;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= D * V) return;
    const int d = e / V;
    size_t base = 0;
    for (int s2 = 0; s2 < seq; ++s2) base += (cu_seqlens[s2 + 1] - cu_seqlens[s2] + chunk_len - 1) / chunk_len;
    const int n_chunks = (cu_seqlens[seq + 1] - cu_seqlens[seq] + chunk_len - 1) / chunk_len;
    float* sp = state + ((size_t)slot * H + h) * D * V + e;
    float S = *sp;
    for (int cnk = 0; cnk < n_chunks; ++cnk) {
        float* cs = chunk_state + ((base + cnk) * H + h) * D * V + e;
        const float add = *cs;
        *cs = S;
        S = fmaf(chunk_decay[((base + cnk) * H + h) * D + d], S, add);
    }
    *sp = S;
}

template <typename T>
static int launch_decay_scan(const void* qk, const void* vsrc, const void* raw, float* out, float* state, float* chunk_state,
                             float* chunk_decay, RecArgs a, int n_seqs, int threads, size_t smem, int max_chunks,
                             cudaStream_t stream) {
    const dim3 grid(a.H * a.v_blocks, n_seqs, max_chunks > 0 ? max_chunks : 1), block(threads);
    cudaError_t e = cudaSuccess;
#define BFI_REC_LAUNCH(PH)                                                                                               \
    do {                                                                                                                 \
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(decay_scan_kernel<T, PH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e == cudaSuccess)                                                                                            \
            bfi_launch(decay_scan_kernel<T, PH>, grid, block, smem, stream, (const T*)qk, (const T*)vsrc, (const T*)raw, out, state,     \
                       chunk_state, chunk_decay, a);                                                                     \
    } while (0)
    if (max_chunks <= 0) {
        BFI_REC_LAUNCH(0);
    } else {
        BFI_REC_LAUNCH(1);
        if (e == cudaSuccess) {
            const int per = a.D * a.V;
            bfi_launch(decay_chunk_carry_kernel, dim3((per + 255) / 256, a.H, n_seqs), dim3(256), 0, stream, state, chunk_state,
                       (const float*)chunk_decay, a.cu_seqlens, a.seq_slot, a.H, a.D, a.V, a.chunk_len);
            BFI_REC_LAUNCH(3);
        }
    }
#undef BFI_REC_LAUNCH
    if (e != cudaSuccess) return bfi_fail("decay_scan: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    return bfi_check_launch("decay_scan");
}

template <typename T, int MODE, int DMAX>
static void launch_regs_phases(const void* qk, const void* vsrc, const void* raw, float* out, float* state, float* chunk_state,
                               float* chunk_decay, const RecArgs& a, int n_seqs, int max_chunks, cudaStream_t stream) {
    const dim3 grid(a.H * a.v_blocks, n_seqs, max_chunks > 0 ? max_chunks : 1), block(REC_WARPS * 32);
    if (max_chunks <= 0) {
        bfi_launch(decay_scan_regs_kernel<T, 0, MODE, DMAX>, grid, block, 0, stream, (const T*)qk, (const T*)vsrc, (const T*)raw, out,
                   state, chunk_state, chunk_decay, a);
        return;
    }
    bfi_launch(decay_scan_regs_kernel<T, 1, MODE, DMAX>, grid, block, 0, stream, (const T*)qk, (const T*)vsrc, (const T*)raw, out,
               state, chunk_state, chunk_decay, a);
    const int per = a.D * a.V;
    bfi_launch(decay_chunk_carry_kernel, dim3((per + 255) / 256, a.H, n_seqs), dim3(256), 0, stream, state, chunk_state,
               (const float*)chunk_decay, a.cu_seqlens, a.seq_slot, a.H, a.D, a.V, a.chunk_len);
    bfi_launch(decay_scan_regs_kernel<T, 3, MODE, DMAX>, grid, block, 0, stream, (const T*)qk, (const T*)vsrc, (const T*)raw, out,
               state, chunk_state, chunk_decay, a);
}

template <typename T>
static int launch_decay_scan_regs(const void* qk, const void* vsrc, const void* raw, float* out, float* state,
                                  float* chunk_state, float* chunk_decay, RecArgs a, int n_seqs, int max_chunks,
                                  cudaStream_t stream) {
    a.vb = REC_WARPS * 32, a.v_blocks = (a.V + REC_WARPS * 32 - 1) / (REC_WARPS * 32);     // a block per 128 columns
#define BFI_REC_REGS(M, DM) \
    launch_regs_phases<T, M, DM>(qk, vsrc, raw, out, state, chunk_state, chunk_decay, a, n_seqs, max_chunks, stream)
    if (a.mode == REC_DECAY_STEP) {
        if (a.D <= 32) BFI_REC_REGS(REC_DECAY_STEP, 32);
        else if (a.D <= 64) BFI_REC_REGS(REC_DECAY_STEP, 64);
        else BFI_REC_REGS(REC_DECAY_STEP, 128);
    } else {
        if (a.D <= 32) BFI_REC_REGS(REC_DECAY_SIGMOID, 32);
        else if (a.D <= 64) BFI_REC_REGS(REC_DECAY_SIGMOID, 64);
        else BFI_REC_REGS(REC_DECAY_SIGMOID, 128);
    }
#undef BFI_REC_REGS
    return bfi_check_launch("decay_scan");
}

// Tests set this to run the general kernels (the state in shared memory) at sizes the register
// kernels would take.
static int g_rec_general = 0;
extern "C" int bfi_decay_scan_general(int on) {
    g_rec_general = on ? 1 : 0;
    return 0;
}

// `chunk_len` > 0 runs the chunked form: `chunk_state` then holds H * D * V floats and `chunk_decay`
// H * D floats for every chunk of the step (sum over the sequences of ceil(tokens / chunk_len), at
// most n_tokens / chunk_len + n_seqs), and `max_chunks` is the most chunks one sequence has.
extern "C" int bfi_decay_scan(const void* qk, long qk_stride, int q_off, int k_off, const void* vsrc, long v_stride,
                              int v_off, const void* raw, long r_stride, int r_off, int dtype, float* out,
                              long out_stride, float* state, const int* cu_seqlens, const int* seq_slot, int n_seqs,
                              int H, int D, int V, int heads_per_group, int mode, float q_scale, float inv_tau,
                              const float* bias, const float* rate, const float* skip, int few_tokens, int chunk_len,
                              int max_chunks, float* chunk_state, float* chunk_decay, cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(dtype), "decay_scan: unknown dtype code %d", dtype);
    BFI_REQUIRE(H > 0 && D > 0 && V > 0, "decay_scan: bad sizes heads=%d dim=%d vdim=%d", H, D, V);
    BFI_REQUIRE(heads_per_group > 0 && H % heads_per_group == 0, "decay_scan: %d heads do not form groups of %d", H,
                heads_per_group);
    BFI_REQUIRE(mode == REC_DECAY_STEP || mode == REC_DECAY_SIGMOID, "decay_scan: unknown decay form %d", mode);
    BFI_REQUIRE(bias != nullptr && (mode != REC_DECAY_STEP || rate != nullptr), "decay_scan: the decay's constants are missing");
    BFI_REQUIRE(out_stride >= (long)H * V, "decay_scan: output stride shorter than the heads");
    BFI_REQUIRE(chunk_len == 0 || (chunk_len > 0 && max_chunks > 0 && max_chunks <= 65535 && chunk_state && chunk_decay),
                "decay_scan: the chunked form needs its chunk length, count and scratch");
    if (n_seqs <= 0) return 0;
    RecArgs a;
    a.qk_stride = qk_stride, a.v_stride = v_stride, a.r_stride = r_stride, a.out_stride = out_stride;
    a.q_off = q_off, a.k_off = k_off, a.v_off = v_off, a.r_off = r_off;
    a.H = H, a.D = D, a.V = V, a.heads_per_group = heads_per_group, a.mode = mode;
    a.q_scale = q_scale, a.inv_tau = inv_tau, a.bias = bias, a.rate = rate, a.skip = skip;
    a.cu_seqlens = cu_seqlens, a.seq_slot = seq_slot, a.chunk_len = chunk_len;
    if (few_tokens == 2 && D <= REC_STEP_DMAX && !g_rec_general && n_seqs <= 65535) {
        // every sequence brings exactly one token
        if (dtype == BFI_F32) return launch_decay_step<float>(qk, vsrc, raw, out, state, a, n_seqs, stream);
        return launch_decay_step<bf16>(qk, vsrc, raw, out, state, a, n_seqs, stream);
    }
    if (D <= 128 && !g_rec_general && (long)H * ((V + 31) / 32) <= 2147483647L && n_seqs <= 65535) {
        // the state in registers, a warp per 32 columns
        const int chunks_r = chunk_len > 0 ? max_chunks : 0;
        if (dtype == BFI_F32)
            return launch_decay_scan_regs<float>(qk, vsrc, raw, out, state, chunk_state, chunk_decay, a, n_seqs, chunks_r, stream);
        return launch_decay_scan_regs<bf16>(qk, vsrc, raw, out, state, chunk_state, chunk_decay, a, n_seqs, chunks_r, stream);
    }
    // columns per block: few where the step is short (more blocks share the state's traffic)
    int vb = V;
    const int want = few_tokens ? 16 : 32;      // few_tokens: 1 = no sequence brings more than one token, 2 = each brings exactly one
    if (V > want) vb = want;
    const int v_blocks = (V + vb - 1) / vb;
    int threads = vb * (256 / vb > 0 ? 256 / vb : 1);
    if (threads < 32) threads = vb * ((32 + vb - 1) / vb);
    a.vb = vb, a.v_blocks = v_blocks;
    BFI_REQUIRE((long)H * v_blocks <= 2147483647L && n_seqs <= 65535, "decay_scan: too many heads or sequences for one launch");
    const size_t smem = ((size_t)D * vb + 4 * (size_t)D + threads) * sizeof(float);
    BFI_REQUIRE(smem <= 200 * 1024, "decay_scan: a state tile of %d x %d does not fit shared memory", D, vb);
    const int chunks = chunk_len > 0 ? max_chunks : 0;
    if (dtype == BFI_F32)
        return launch_decay_scan<float>(qk, vsrc, raw, out, state, chunk_state, chunk_decay, a, n_seqs, threads, smem, chunks, stream);
    return launch_decay_scan<bf16>(qk, vsrc, raw, out, state, chunk_state, chunk_decay, a, n_seqs, threads, smem, chunks, stream);
}

// ------------------------------------------------------------------------------------------
// Causal convolution per channel.  Token t of a sequence reads its own input and the taps-1
// before it: rows of this step while they belong to the same sequence, then the kept inputs of
// earlier steps (state [slots][taps-1][C], oldest first; zero when the slot was taken, which is
// what stands before a sequence's first token).
//     y[t, c] = act(bias[c] + sum_j w[c, taps-1-j] * u[t-j, c])      act: silu (1) or none (0)
// Options, each a pointer or flag that may be absent:
//   add_input   y[t, c] += u[t, c]  (the convolution as a correction of its own input)
//   copy        copy[t, c] = u[t, c] in the output type (the input itself, for a reader beside the
//               convolution that wants it in the product's type)
//   mix         for channels c >= mix_off, with e = c - mix_off:
//                   mix_src:  y[t, c] = (1 - lambda) y[t, c] + lambda mix_src[t, e]
//                   mix_dst:  mix_dst[t, e] = y[t, c]       (after the mixing, when both are there)
//               lambda is one float32 on the device.
// The input may be float32 while the output is bfloat16 (a convolution straight off the residual
// stream).  conv_forward_kernel computes y; conv_keep_kernel then moves the state on (it must not
// run before every y of the step has read the old state: it is a launch of its own).  When every
// sequence brings one token, one thread does both for its channel.
// ------------------------------------------------------------------------------------------
struct ConvExtras {
    int act, add_input;
    void* copy;
    long copy_stride;
    int mix_off;
    const void* mix_src;
    void* mix_dst;
    long mix_stride;
    const float* mix_lambda;
};

template <typename TI, typename TO>
__global__ void conv_forward_kernel(const TI* __restrict__ u, long u_stride, int u_off, const void* __restrict__ w,
                                    const void* __restrict__ bias, int w_dtype, float* __restrict__ state,
                                    TO* __restrict__ y, long y_stride, const int* __restrict__ token_slot, int C, int taps,
                                    int fused_keep, const ConvExtras x) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int ch = blockIdx.y * blockDim.x + threadIdx.x;
    const int slot = token_slot[t];
    if (slot < 0 || ch >= C) return;
    int own = 0;                                   // rows before t that belong to the same sequence
    while (own < taps - 1 && t - own - 1 >= 0 && token_slot[t - own - 1] == slot) ++own;
    float* st = state + (size_t)slot * (taps - 1) * C + ch;
    float in[REC_MAX_TAPS];
    float acc = bias ? load_as_f32(bias, w_dtype, ch) : 0.0f;
    for (int j = 0; j < taps; ++j) {
        in[j] = j <= own ? to_f32(u[(size_t)(t - j) * u_stride + u_off + ch])
                         : st[(size_t)(taps - 1 + own - j) * C];
        acc = fmaf(load_as_f32(w, w_dtype, (size_t)ch * taps + (taps - 1 - j)), in[j], acc);
    }
    if (x.act) acc = rec_silu(acc);
    if (x.add_input) acc += in[0];
    if (ch >= x.mix_off) {
        const size_t e = (size_t)t * x.mix_stride + (ch - x.mix_off);
        if (x.mix_src != nullptr) {
            const float lam = *x.mix_lambda;
            acc = (1.0f - lam) * acc + lam * to_f32(reinterpret_cast<const TO*>(x.mix_src)[e]);
        }
        if (x.mix_dst != nullptr) reinterpret_cast<TO*>(x.mix_dst)[e] = from_f32<TO>(acc);
    }
    y[(size_t)t * y_stride + ch] = from_f32<TO>(acc);
    if (x.copy != nullptr) reinterpret_cast<TO*>(x.copy)[(size_t)t * x.copy_stride + ch] = from_f32<TO>(in[0]);
    if (fused_keep)                                // one token per sequence: the window moves on by one
        for (int i = 0; i < taps - 1; ++i) st[(size_t)i * C] = in[taps - 2 - i];
}

// The same for bfloat16 outputs when channels, offsets and strides come in whole groups of 8: a thread owns 8
// neighbouring channels of one token, reads every row it needs as 16 (or 32) bytes and writes 16.
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
}
__device__ __forceinline__ void load8(const bf16* p, float (&v)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(h[k]);
        v[2 * k] = f.x, v[2 * k + 1] = f.y;
    }
}
__device__ __forceinline__ void store8(bf16* p, const float (&v)[8]) {
    uint4 packed;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
    *reinterpret_cast<uint4*>(p) = packed;
}

template <typename TI>
__global__ void conv_forward_vec_kernel(const TI* __restrict__ u, long u_stride, int u_off, const void* __restrict__ w,
                                        const void* __restrict__ bias, int w_dtype, float* __restrict__ state,
                                        bf16* __restrict__ y, long y_stride, const int* __restrict__ token_slot, int n_tokens,
                                        int C, int taps, int fused_keep, const ConvExtras x) {
    pdl_trigger();
    pdl_wait();
    const int groups = C >> 3;
    const long total = (long)n_tokens * groups;
    for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long)gridDim.x * blockDim.x) {
        const int t = (int)(idx / groups);
        const int ch = (int)(idx - (long)t * groups) << 3;
        const int slot = token_slot[t];
        if (slot < 0) continue;
        int own = 0;                               // rows before t that belong to the same sequence
        while (own < taps - 1 && t - own - 1 >= 0 && token_slot[t - own - 1] == slot) ++own;
        float* st = state + (size_t)slot * (taps - 1) * C + ch;
        float acc[8], cur[8], in[8], prev[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] = bias ? load_as_f32(bias, w_dtype, ch + k) : 0.0f;
        for (int j = 0; j < taps; ++j) {
            float* place = st + (size_t)(taps - 1 + own - j) * C;      // where the input j steps back is kept, if it is
            if (j <= own)
                load8(u + (size_t)(t - j) * u_stride + u_off + ch, in);
            else
                load8(place, in);
            if (j == 0) {
#pragma unroll
                for (int k = 0; k < 8; ++k) cur[k] = in[k];
            }
#pragma unroll
            for (int k = 0; k < 8; ++k)
                acc[k] = fmaf(load_as_f32(w, w_dtype, (size_t)(ch + k) * taps + (taps - 1 - j)), in[k], acc[k]);
            if (fused_keep) {
                // one token per sequence (own is 0): the window moves on by one, so the input j - 1 steps back takes
                // the place that has just been read
                if (j >= 1) {
                    reinterpret_cast<float4*>(place)[0] = make_float4(prev[0], prev[1], prev[2], prev[3]);
                    reinterpret_cast<float4*>(place)[1] = make_float4(prev[4], prev[5], prev[6], prev[7]);
                }
#pragma unroll
                for (int k = 0; k < 8; ++k) prev[k] = in[k];
            }
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            if (x.act) acc[k] = rec_silu(acc[k]);
            if (x.add_input) acc[k] += cur[k];
        }
        if (ch >= x.mix_off) {
            const size_t e = (size_t)t * x.mix_stride + (ch - x.mix_off);
            if (x.mix_src != nullptr) {
                const float lam = *x.mix_lambda;
                float other[8];
                load8(reinterpret_cast<const bf16*>(x.mix_src) + e, other);
#pragma unroll
                for (int k = 0; k < 8; ++k) acc[k] = (1.0f - lam) * acc[k] + lam * other[k];
            }
            if (x.mix_dst != nullptr) store8(reinterpret_cast<bf16*>(x.mix_dst) + e, acc);
        }
        store8(y + (size_t)t * y_stride + ch, acc);
        if (x.copy != nullptr) store8(reinterpret_cast<bf16*>(x.copy) + (size_t)t * x.copy_stride + ch, cur);
    }
}

// The same again for 2 to 4 taps: a thread owns 8 neighbouring channels of CONV_TOK consecutive tokens, holds its
// weights in registers and reads its tokens' rows and the TAPS - 1 rows before them once, all loads in flight
// together, so a row is read once per thread instead of once per tap; a tap that reaches back past the rows of
// the token's own sequence reads the kept inputs instead.
#define CONV_TOK 4

template <typename TI, int TAPS>
__global__ void __launch_bounds__(128)
conv_forward_win_kernel(const TI* __restrict__ u, long u_stride, int u_off, const void* __restrict__ w,
                        const void* __restrict__ bias, int w_dtype, float* __restrict__ state, bf16* __restrict__ y,
                        long y_stride, const int* __restrict__ token_slot, int n_tokens, int C, int fused_keep,
                        const ConvExtras x) {
    pdl_trigger();
    const int groups = C >> 3;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const long tile = idx / groups;
    const int ch = (int)(idx - tile * groups) << 3;
    const bool live = tile * CONV_TOK < n_tokens;
    float wt[TAPS][8], bs[8];                      // wt[j]: the weight of the input j steps back
    if (live) {
        // the 8 channels' taps lie side by side in the weights: 8 * TAPS values, read 16 bytes at a time
        float flat[8 * TAPS];
        if (w_dtype == BFI_BF16) {
            const bf16* p = reinterpret_cast<const bf16*>(w) + (size_t)ch * TAPS;
#pragma unroll
            for (int q = 0; q < TAPS; ++q) {
                float part[8];
                load8(p + 8 * q, part);
#pragma unroll
                for (int k = 0; k < 8; ++k) flat[8 * q + k] = part[k];
            }
        } else {
            const float* p = reinterpret_cast<const float*>(w) + (size_t)ch * TAPS;
#pragma unroll
            for (int q = 0; q < TAPS; ++q) {
                float part[8];
                load8(p + 8 * q, part);
#pragma unroll
                for (int k = 0; k < 8; ++k) flat[8 * q + k] = part[k];
            }
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            bs[k] = bias ? load_as_f32(bias, w_dtype, ch + k) : 0.0f;
#pragma unroll
            for (int j = 0; j < TAPS; ++j) wt[j][k] = flat[k * TAPS + (TAPS - 1 - j)];
        }
    }
    pdl_wait();
    if (!live) return;
    // the slots of the tile's rows and of the TAPS - 1 rows before them, then all those rows at once: no load
    // waits for another
    constexpr int ROWS = CONV_TOK + TAPS - 1;
    const int t0 = (int)tile * CONV_TOK;
    int sl[ROWS];
    float rows[ROWS][8];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const int tt = t0 - (TAPS - 1) + r;
        sl[r] = (tt >= 0 && tt < n_tokens) ? token_slot[tt] : -1;
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const int tt = t0 - (TAPS - 1) + r;
        if (sl[r] >= 0) load8(u + (size_t)tt * u_stride + u_off + ch, rows[r]);
    }
#pragma unroll
    for (int i = 0; i < CONV_TOK; ++i) {
        const int ri = i + TAPS - 1;
        const int t = t0 + i;
        const int slot = sl[ri];
        if (slot < 0) continue;                    // padding, or past the step's tokens
        float* st = state + (size_t)slot * (TAPS - 1) * C + ch;
        int own = 0;                               // rows before t that belong to the same sequence
#pragma unroll
        for (int j = 1; j < TAPS; ++j)
            if (own == j - 1 && sl[ri - j] == slot) own = j;
        float acc[8], kept[TAPS][8];               // kept[j]: the input j steps back, where it comes from the state
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] = bs[k];
#pragma unroll
        for (int j = 0; j < TAPS; ++j) {
            if (j <= own) {
#pragma unroll
                for (int k = 0; k < 8; ++k) acc[k] = fmaf(wt[j][k], rows[ri - j][k], acc[k]);
            } else {
                load8(st + (size_t)(TAPS - 1 + own - j) * C, kept[j]);
#pragma unroll
                for (int k = 0; k < 8; ++k) acc[k] = fmaf(wt[j][k], kept[j][k], acc[k]);
            }
        }
        if (fused_keep) {
            // one token per sequence: the window moves on by one, after every place of it has been read
#pragma unroll
            for (int j = 0; j < TAPS - 1; ++j) {
                float* dst = st + (size_t)(TAPS - 2 - j) * C;
                const float* src = j <= own ? rows[ri - j] : kept[j];
                reinterpret_cast<float4*>(dst)[0] = make_float4(src[0], src[1], src[2], src[3]);
                reinterpret_cast<float4*>(dst)[1] = make_float4(src[4], src[5], src[6], src[7]);
            }
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            if (x.act) acc[k] = rec_silu(acc[k]);
            if (x.add_input) acc[k] += rows[ri][k];
        }
        if (ch >= x.mix_off) {
            const size_t e = (size_t)t * x.mix_stride + (ch - x.mix_off);
            if (x.mix_src != nullptr) {
                const float lam = *x.mix_lambda;
                float other[8];
                load8(reinterpret_cast<const bf16*>(x.mix_src) + e, other);
#pragma unroll
                for (int k = 0; k < 8; ++k) acc[k] = (1.0f - lam) * acc[k] + lam * other[k];
            }
            if (x.mix_dst != nullptr) store8(reinterpret_cast<bf16*>(x.mix_dst) + e, acc);
        }
        store8(y + (size_t)t * y_stride + ch, acc);
        if (x.copy != nullptr) store8(reinterpret_cast<bf16*>(x.copy) + (size_t)t * x.copy_stride + ch, rows[ri]);
    }
}

template <typename TI, int TAPS>
static void launch_conv_win(const void* u, long u_stride, int u_off, const void* w, const void* bias, int w_dtype, float* state,
                            void* y, long y_stride, const int* token_slot, int n_tokens, int C, int fused, const ConvExtras& x,
                            cudaStream_t stream) {
    const long total = (long)((n_tokens + CONV_TOK - 1) / CONV_TOK) * (C / 8);
    bfi_launch(conv_forward_win_kernel<TI, TAPS>, dim3((unsigned)((total + 127) / 128)), dim3(128), 0, stream, (const TI*)u, u_stride,
               u_off, w, bias, w_dtype, state, (bf16*)y, y_stride, token_slot, n_tokens, C, fused, x);
}

template <typename T>
__global__ void conv_keep_kernel(const T* __restrict__ u, long u_stride, int u_off, float* __restrict__ state,
                                 const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot, int C, int taps) {
    pdl_trigger();
    pdl_wait();
    const int seq = blockIdx.x;
    const int ch = blockIdx.y * blockDim.x + threadIdx.x;
    const int slot = seq_slot[seq];
    if (slot < 0 || ch >= C) return;
    const int t0 = cu_seqlens[seq], n = cu_seqlens[seq + 1] - t0;
    float* st = state + (size_t)slot * (taps - 1) * C + ch;
    float keep[REC_MAX_TAPS];
    for (int i = 0; i < taps - 1; ++i) {
        const int r = n - (taps - 1) + i;          // which of the step's tokens lands in place i
        keep[i] = r >= 0 ? to_f32(u[(size_t)(t0 + r) * u_stride + u_off + ch]) : st[(size_t)(i + n) * C];
    }
    for (int i = 0; i < taps - 1; ++i) st[(size_t)i * C] = keep[i];
}

extern "C" int bfi_causal_conv(const void* u, long u_stride, int u_off, int dtype, const void* w, const void* bias,
                               int w_dtype, float* state, void* y, long y_stride, int y_dtype, const int* token_slot,
                               const int* cu_seqlens, const int* seq_slot, int n_tokens, int n_seqs, int C, int taps,
                               int single_tokens, int act, int add_input, void* copy, long copy_stride, int mix_off,
                               const void* mix_src, void* mix_dst, long mix_stride, const float* mix_lambda,
                               cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(dtype) && dtype_ok(w_dtype) && dtype_ok(y_dtype), "causal_conv: unknown dtype code");
    BFI_REQUIRE(dtype == y_dtype || dtype == BFI_F32, "causal_conv: the output has the input's type, or the input is float32");
    BFI_REQUIRE(C > 0 && taps >= 1 && taps <= REC_MAX_TAPS, "causal_conv: %d channels, %d taps (at most %d)", C, taps, REC_MAX_TAPS);
    BFI_REQUIRE(u_stride >= u_off + C && y_stride >= C, "causal_conv: row stride shorter than the channels");
    BFI_REQUIRE(copy == nullptr || copy_stride >= C, "causal_conv: the copy's row stride is shorter than the channels");
    const bool mixes = mix_src != nullptr || mix_dst != nullptr;
    BFI_REQUIRE(!mixes || (mix_off >= 0 && mix_off < C && mix_stride >= C - mix_off && (mix_src == nullptr || mix_lambda != nullptr)),
                "causal_conv: the mixed channels need rows of their count and, to mix, the factor");
    if (n_tokens <= 0 || n_seqs <= 0) return 0;
    const int threads = 128;
    const dim3 grid_t(n_tokens, (C + threads - 1) / threads), grid_s(n_seqs, (C + threads - 1) / threads);
    BFI_REQUIRE(grid_t.y <= 65535, "causal_conv: %d channels are too many for one launch", C);
    const int fused = single_tokens ? 1 : 0;
    ConvExtras x;
    x.act = act, x.add_input = add_input, x.copy = copy, x.copy_stride = copy_stride;
    x.mix_off = mixes ? mix_off : C, x.mix_src = mix_src, x.mix_dst = mix_dst, x.mix_stride = mix_stride, x.mix_lambda = mix_lambda;
    const auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const bool vec = y_dtype == BFI_BF16 && C % 8 == 0 && u_off % 8 == 0 && u_stride % 8 == 0 && y_stride % 8 == 0 && al16(u) &&
                     al16(y) && al16(state) && (copy == nullptr || (copy_stride % 8 == 0 && al16(copy))) &&
                     (!mixes || (mix_off % 8 == 0 && mix_stride % 8 == 0 && (mix_src == nullptr || al16(mix_src)) &&
                                 (mix_dst == nullptr || al16(mix_dst))));
    if (vec && taps >= 2 && taps <= 4 && al16(w)) {
        const bool f32 = dtype == BFI_F32;
#define BFI_CONV_WIN(TAPS)                                                                                                        \
    if (f32)                                                                                                                      \
        launch_conv_win<float, TAPS>(u, u_stride, u_off, w, bias, w_dtype, state, y, y_stride, token_slot, n_tokens, C, fused, x, \
                                     stream);                                                                                     \
    else                                                                                                                          \
        launch_conv_win<bf16, TAPS>(u, u_stride, u_off, w, bias, w_dtype, state, y, y_stride, token_slot, n_tokens, C, fused, x,  \
                                    stream)
        if (taps == 2) {
            BFI_CONV_WIN(2);
        } else if (taps == 3) {
            BFI_CONV_WIN(3);
        } else {
            BFI_CONV_WIN(4);
        }
#undef BFI_CONV_WIN
    } else if (vec) {
        const long total = (long)n_tokens * (C / 8);
        long blocks = (total + threads - 1) / threads;
        const long most = (long)bfi_sm_count() * 16;
        if (blocks > most) blocks = most;
        if (dtype == BFI_F32)
            bfi_launch(conv_forward_vec_kernel<float>, dim3((unsigned)blocks), dim3(threads), 0, stream, (const float*)u, u_stride, u_off,
                       w, bias, w_dtype, state, (bf16*)y, y_stride, token_slot, n_tokens, C, taps, fused, x);
        else
            bfi_launch(conv_forward_vec_kernel<bf16>, dim3((unsigned)blocks), dim3(threads), 0, stream, (const bf16*)u, u_stride, u_off,
                       w, bias, w_dtype, state, (bf16*)y, y_stride, token_slot, n_tokens, C, taps, fused, x);
    } else
    if (dtype == BFI_F32 && y_dtype == BFI_F32)
        bfi_launch(conv_forward_kernel<float, float>, grid_t, dim3(threads), 0, stream, (const float*)u, u_stride, u_off, w, bias,
                   w_dtype, state, (float*)y, y_stride, token_slot, C, taps, fused, x);
    else if (dtype == BFI_F32)
        bfi_launch(conv_forward_kernel<float, bf16>, grid_t, dim3(threads), 0, stream, (const float*)u, u_stride, u_off, w, bias,
                   w_dtype, state, (bf16*)y, y_stride, token_slot, C, taps, fused, x);
    else
        bfi_launch(conv_forward_kernel<bf16, bf16>, grid_t, dim3(threads), 0, stream, (const bf16*)u, u_stride, u_off, w, bias,
                   w_dtype, state, (bf16*)y, y_stride, token_slot, C, taps, fused, x);
    int rc = bfi_check_launch("causal_conv");
    if (rc || fused || taps == 1) return rc;
    if (dtype == BFI_F32)
        bfi_launch(conv_keep_kernel<float>, grid_s, dim3(threads), 0, stream, (const float*)u, u_stride, u_off, state, cu_seqlens,
                   seq_slot, C, taps);
    else
        bfi_launch(conv_keep_kernel<bf16>, grid_s, dim3(threads), 0, stream, (const bf16*)u, u_stride, u_off, state, cu_seqlens,
                   seq_slot, C, taps);
    return bfi_check_launch("causal_conv (state)");
}

// ------------------------------------------------------------------------------------------
// The gate and the norm after a recurrence.  A row of `width` values is cut into `parts` equal
// parts, each divided by its own root mean square; the weight has `w_len` values and repeats
// along the row (w_len = width: one weight per value; w_len = width / parts: shared by the parts).
//     gate_first:  y = norm_parts(x * act(gate)) * w          otherwise:  y = norm_parts(x) * w * act(gate)
// act is sigmoid (0) or silu (1).  x float32; gate and y in the activation storage type.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void gated_group_norm_kernel(const float* __restrict__ x, long x_stride, const T* __restrict__ gate,
                                        long gate_stride, const void* __restrict__ w, int w_dtype, int w_len,
                                        T* __restrict__ y, long y_stride, int width, int parts, int gate_first,
                                        int gate_act, float eps) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int len = width / parts;
    const float* xr = x + (size_t)t * x_stride;
    const T* gr = gate + (size_t)t * gate_stride;
    T* yr = y + (size_t)t * y_stride;
    for (int p = warp; p < parts; p += n_warps) {
        const int j0 = p * len;
        float ss = 0.0f;
        for (int j = lane; j < len; j += 32) {
            float v = xr[j0 + j];
            if (gate_first) {
                const float gv = to_f32(gr[j0 + j]);
                v *= gate_act ? rec_silu(gv) : rec_sigmoid(gv);
            }
            ss = fmaf(v, v, ss);
        }
        ss = warp_sum(ss);
        const float scale = 1.0f / sqrtf(ss / (float)len + eps);
        for (int j = lane; j < len; j += 32) {
            const float gv = to_f32(gr[j0 + j]);
            const float ga = gate_act ? rec_silu(gv) : rec_sigmoid(gv);
            yr[j0 + j] = from_f32<T>(xr[j0 + j] * ga * scale * load_as_f32(w, w_dtype, (j0 + j) % w_len));
        }
    }
}

extern "C" int bfi_gated_group_norm(const float* x, long x_stride, const void* gate, long gate_stride, int dtype,
                                    const void* w, int w_dtype, int w_len, void* y, long y_stride, int n_rows, int width,
                                    int parts, int gate_first, int gate_act, float eps, cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(dtype) && dtype_ok(w_dtype), "gated_group_norm: unknown dtype code");
    BFI_REQUIRE(n_rows >= 0 && width > 0 && parts > 0 && width % parts == 0,
                "gated_group_norm: a row of %d values does not cut into %d equal parts", width, parts);
    BFI_REQUIRE(w_len > 0 && width % w_len == 0, "gated_group_norm: a weight of %d values does not repeat along %d", w_len, width);
    BFI_REQUIRE(x_stride >= width && gate_stride >= width && y_stride >= width, "gated_group_norm: row stride shorter than the row");
    if (n_rows == 0) return 0;
    int warps = parts < 8 ? parts : 8;
    if (dtype == BFI_F32)
        bfi_launch(gated_group_norm_kernel<float>, dim3(n_rows), dim3(32 * warps), 0, stream, x, x_stride, (const float*)gate,
                   gate_stride, w, w_dtype, w_len, (float*)y, y_stride, width, parts, gate_first, gate_act, eps);
    else
        bfi_launch(gated_group_norm_kernel<bf16>, dim3(n_rows), dim3(32 * warps), 0, stream, x, x_stride, (const bf16*)gate,
                   gate_stride, w, w_dtype, w_len, (bf16*)y, y_stride, width, parts, gate_first, gate_act, eps);
    return bfi_check_launch("gated_group_norm");
}

BFI_TRACE_EXPORT(recurrence)
