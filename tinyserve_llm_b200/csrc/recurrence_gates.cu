// What enters the scan of linear_recurrence.cu for two recurrences whose gates are computed from the
// input: the gated delta rule and the matrix memory with exponential gates (mLSTM).  Everything here
// is float32; the inputs are projections' outputs in the activation dtype (or float32).
//
// Gated delta rule.  q and k ([tokens, kv_heads * dim], float32, after their short convolution) become
// unit vectors per head, x / sqrt(sum(x^2) + unit_eps), q also times q_scale; value head h uses q/k
// head h / (heads / kv_heads).  The decay of head h, key channel i is
//   a = exp(-exp(A_log[h]) * softplus(z[t, h, i] + dt_bias[h, i])),   beta[t, h] = sigmoid(b[t, h]).
//
// Matrix memory.  Per head (x_i, x_f: float32 projections), log input gate i = cap tanh((x_i + b_i) / cap), log forget gate
// f = log_sigmoid(cap tanh((x_f + b_f) / cap)), running maximum m_t = max(f + m_(t-1), i) carried in the
// request's state (it starts at 0); the scan then runs with decay exp(f + m_(t-1) - m_t) for all of a
// head's key channels, k times exp(i - m_t), and q times q_scale.  m_t goes out per token for the read-out.
#include "common.cuh"

__device__ __forceinline__ float softplus(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float log_sigmoid_f(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// one warp a (token, head)
template <typename T>
__global__ void delta_prepare_kernel(const float* __restrict__ q, const float* __restrict__ k, long long qk_stride,
                                     const float* __restrict__ z, const float* __restrict__ dt_bias,
                                     const float* __restrict__ a_log, const T* __restrict__ b, long long b_stride,
                                     float* __restrict__ prepared, float* __restrict__ beta, long long items, long long total,
                                     int heads, int kv_heads, int dim, float unit_eps, float q_scale) {
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= items) return;
    const int lane = threadIdx.x & 31;
    const long long t = item / heads;
    const int h = (int)(item % heads), g = h / (heads / kv_heads);
    const float* qr = q + t * qk_stride + (long long)g * dim;
    const float* kr = k + t * qk_stride + (long long)g * dim;
    float sq = 0.f, sk = 0.f;
    for (int i = lane; i < dim; i += 32) { sq += qr[i] * qr[i]; sk += kr[i] * kr[i]; }
    const float inv_q = q_scale / sqrtf(warp_sum(sq) + unit_eps), inv_k = 1.f / sqrtf(warp_sum(sk) + unit_eps);
    const float rate = expf(a_log[h]);
    const long long at = item * dim;
    for (int i = lane; i < dim; i += 32) {
        prepared[at + i] = qr[i] * inv_q;
        prepared[total + at + i] = kr[i] * inv_k;
        prepared[2 * total + at + i] = expf(-rate * softplus(z[at + i] + dt_bias[(long long)h * dim + i]));
    }
    if (lane == 0) beta[item] = 1.f / (1.f + expf(-to_float<T>(b[t * b_stride + h])));
}

TS_API int ts_delta_prepare(const float* q, const float* k, long long qk_stride, const float* z, const float* dt_bias,
                            const float* a_log, const void* b, long long b_stride, float* prepared, float* beta,
                            int num_tokens, int heads, int kv_heads, int dim, float unit_eps, float q_scale, int dtype,
                            cudaStream_t stream) {
    TS_REQUIRE(heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dim > 0, "delta_prepare: %d heads over %d q/k heads",
               heads, kv_heads);
    if (num_tokens <= 0) return 0;
    const long long items = (long long)num_tokens * heads, total = items * dim;
    const unsigned blocks = (unsigned)((items + 3) / 4);
    if (dtype == TS_F32)
        delta_prepare_kernel<float><<<blocks, 128, 0, stream>>>(q, k, qk_stride, z, dt_bias, a_log, (const float*)b, b_stride,
            prepared, beta, items, total, heads, kv_heads, dim, unit_eps, q_scale);
    else if (dtype == TS_BF16)
        delta_prepare_kernel<__nv_bfloat16><<<blocks, 128, 0, stream>>>(q, k, qk_stride, z, dt_bias, a_log,
            (const __nv_bfloat16*)b, b_stride, prepared, beta, items, total, heads, kv_heads, dim, unit_eps, q_scale);
    else
        return ts_fail("delta_prepare: unknown dtype code %d", dtype);
    TS_LAUNCH_CHECK("delta_prepare");
    return 0;
}

// One warp a (request, head): 32 tokens at a time, each lane its token's gates; the running maximum is carried
// through the lanes by a scan.  factors[0] = decay, factors[1] = the key's factor, each [tokens, heads].
__global__ void mlstm_gates_kernel(const float* __restrict__ gi, const float* __restrict__ gf, long long gate_stride,
                                   const float* __restrict__ bias_i, const float* __restrict__ bias_f, float cap,
                                   const int* __restrict__ cu_q, const int* __restrict__ slots, float* __restrict__ state,
                                   long long slot_stride, float* __restrict__ log_max, float* __restrict__ factors,
                                   long long num_items, int num_seqs, int heads) {
    const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= num_seqs * heads) return;
    const int lane = threadIdx.x & 31;
    const int seq = item / heads, h = item % heads;
    const int slot = slots[seq];
    const int begin = cu_q[seq], end = cu_q[seq + 1];
    if (slot < 0 || end <= begin) return;
    float* m_state = state + (long long)slot * slot_stride + h;
    float m = *m_state;
    const float bi = bias_i[h], bf = bias_f[h];
    // a round's projections are loaded one round ahead of their use
    float next_i = begin + lane < end ? gi[(long long)(begin + lane) * gate_stride + h] : 0.f;
    float next_f = begin + lane < end ? gf[(long long)(begin + lane) * gate_stride + h] : 0.f;
    for (int t0 = begin; t0 < end; t0 += 32) {
        const int t = t0 + lane;
        const float raw_i = next_i, raw_f = next_f;
        if (t + 32 < end) {
            next_i = gi[(long long)(t + 32) * gate_stride + h];
            next_f = gf[(long long)(t + 32) * gate_stride + h];
        }
        float i_gate = 0.f, f_gate = 0.f;
        if (t < end) {
            i_gate = cap * tanhf((raw_i + bi) / cap);
            f_gate = log_sigmoid_f(cap * tanhf((raw_f + bf) / cap));
        }
        // m_t = max(f_t + m_(t-1), i_t) is the composition of the maps x -> max(x + a, b); an inclusive scan over the
        // lanes composes them: (a, b) after (a', b') = (a' + a, max(b' + a, b)).  Lanes past the end hold the identity.
        float a = t < end ? f_gate : 0.f, b = t < end ? i_gate : -INFINITY;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float pa = __shfl_up_sync(0xffffffffu, a, o), pb = __shfl_up_sync(0xffffffffu, b, o);
            if (lane >= o) { b = fmaxf(pb + a, b); a = pa + a; }
        }
        const float after = fmaxf(m + a, b);
        float before = __shfl_up_sync(0xffffffffu, after, 1);
        if (lane == 0) before = m;
        m = __shfl_sync(0xffffffffu, after, 31);          // lanes past the end carry the last token's value on
        if (t < end) {
            const long long at = (long long)t * heads + h;
            log_max[at] = after;
            factors[at] = expf(f_gate + before - after);
            factors[num_items + at] = expf(i_gate - after);
        }
    }
    if (lane == 0) *m_state = m;
}

template <typename T>
__global__ void mlstm_prepare_kernel(const T* __restrict__ q, const T* __restrict__ k, long long q_stride, long long k_stride,
                                     const float* __restrict__ factors, long long num_items, float q_scale,
                                     float* __restrict__ prepared, long long total, int heads, int dim) {
    const int width = heads * dim;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const long long t = e / width;
        const int c = (int)(e % width), h = c / dim;
        const long long item = t * heads + h;
        prepared[e] = to_float<T>(q[t * q_stride + c]) * q_scale;
        prepared[total + e] = to_float<T>(k[t * k_stride + c]) * factors[num_items + item];
        prepared[2 * total + e] = factors[item];
    }
}

// `state` points at the request slots' running maxima ([heads] floats a slot, `slot_stride` floats apart).
TS_API int ts_mlstm_prepare(const void* q, const void* k, long long q_stride, long long k_stride, const float* gi,
                            const float* gf, long long gate_stride, const float* bias_i, const float* bias_f, float cap,
                            float q_scale, const int* cu_q, const int* slots, int num_seqs, float* state,
                            long long slot_stride, float* log_max, float* factors, float* prepared, int num_tokens,
                            int heads, int dim, int dtype, cudaStream_t stream) {
    TS_REQUIRE(heads > 0 && dim > 0 && cap > 0.f, "mlstm_prepare: bad sizes or gate cap");
    if (num_tokens <= 0 || num_seqs <= 0) return 0;
    const long long items = (long long)num_tokens * heads, total = items * dim;
    const unsigned blocks_a = (unsigned)(((long long)num_seqs * heads + 3) / 4);
    const unsigned blocks_b = (unsigned)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
#define TS_MLSTM(TYPE)                                                                                                 \
    do {                                                                                                               \
        mlstm_gates_kernel<<<blocks_a, 128, 0, stream>>>(gi, gf, gate_stride, bias_i,                                  \
            bias_f, cap, cu_q, slots, state, slot_stride, log_max, factors, items, num_seqs, heads);                   \
        mlstm_prepare_kernel<TYPE><<<blocks_b, 256, 0, stream>>>((const TYPE*)q, (const TYPE*)k, q_stride, k_stride,   \
            factors, items, q_scale, prepared, total, heads, dim);                                                     \
    } while (0)
    if (dtype == TS_F32) TS_MLSTM(float);
    else if (dtype == TS_BF16) TS_MLSTM(__nv_bfloat16);
    else return ts_fail("mlstm_prepare: unknown dtype code %d", dtype);
#undef TS_MLSTM
    TS_LAUNCH_CHECK("mlstm_prepare");
    return 0;
}
