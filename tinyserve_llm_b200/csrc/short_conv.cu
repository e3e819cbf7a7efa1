// Short causal convolution over time, one filter per channel, followed by silu:
//
//   y[t, c] = silu( sum_{j < taps} w[c, j] * x[t - (taps - 1 - j), c] )        zeros before the sequence's start
//
// The last taps - 1 inputs of a request are part of its state (float32, [taps - 1][channels] in the
// request's slot, oldest first), so a prompt may be cut anywhere and decoding is the same kernel: an
// input from before this step's first token is read from the slot.  A second kernel, launched behind
// the first, moves the slot on.  Sums are float32; the output is float32.
#include "common.cuh"

// grid: (channel blocks, groups of `group` tokens); a CTA's threads are neighbouring channels, each walks the group's
// tokens (8 in a step of many tokens, 1 in a small step, where the walk would only lengthen the step)

template <typename T>
__global__ void short_conv_silu_kernel(const T* __restrict__ x, long long x_stride, const float* __restrict__ w,
                                       const int* __restrict__ seq_of_token, const int* __restrict__ cu_q,
                                       const int* __restrict__ slots, const float* __restrict__ state, long long slot_stride,
                                       float* __restrict__ y, int num_tokens, int channels, int taps, int group) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int t_end = min(num_tokens, (int)(blockIdx.y + 1) * group);
    const float* wc = w + (long long)c * taps;
    for (int t = blockIdx.y * group; t < t_end; ++t) {
        const int seq = seq_of_token[t];
        if (seq < 0) { y[(long long)t * channels + c] = 0.f; continue; }      // a padding row
        const int slot = slots[seq];
        const int begin = cu_q[seq];
        const float* st = state + (long long)slot * slot_stride;
        float acc = 0.f;
        for (int j = 0; j < taps; ++j) {
            const int src = t - begin - (taps - 1 - j);    // token of this step, or (negative) one of the slot's
            float v;
            if (src >= 0) v = to_float<T>(x[(long long)(begin + src) * x_stride + c]);
            else v = slot >= 0 ? st[(long long)(taps - 1 + src) * channels + c] : 0.f;
            acc = fmaf(wc[j], v, acc);
        }
        y[(long long)t * channels + c] = acc / (1.f + expf(-acc));
    }
}

// state <- the last taps - 1 inputs after this step; one thread a (request, channel), oldest entry first, so an
// entry is read before it is overwritten
template <typename T>
__global__ void short_conv_advance_kernel(const T* __restrict__ x, long long x_stride, const int* __restrict__ cu_q,
                                          const int* __restrict__ slots, float* __restrict__ state, long long slot_stride,
                                          int num_seqs, int channels, int taps) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)num_seqs * channels) return;
    const int seq = (int)(idx / channels), c = (int)(idx % channels);
    const int slot = slots[seq];
    const int begin = cu_q[seq], n = cu_q[seq + 1] - begin;
    if (slot < 0 || n <= 0) return;
    float* st = state + (long long)slot * slot_stride;
    for (int i = 0; i < taps - 1; ++i) {
        const int src = n - (taps - 1) + i;
        st[(long long)i * channels + c] = src >= 0 ? to_float<T>(x[(long long)(begin + src) * x_stride + c])
                                                   : st[(long long)(i + n) * channels + c];
    }
}

TS_API int ts_short_conv_silu(const void* x, long long x_stride, const float* w, const int* seq_of_token, const int* cu_q,
                              const int* slots, int num_seqs, float* state, long long slot_stride, float* y, int num_tokens,
                              int channels, int taps, int dtype, cudaStream_t stream) {
    TS_REQUIRE(num_tokens >= 0 && channels > 0 && taps > 0, "short_conv: bad sizes");
    TS_REQUIRE(slot_stride >= (long long)(taps - 1) * channels, "short_conv: a state slot is too small");
    if (num_tokens == 0 || num_seqs == 0) return 0;
    const int group = num_tokens >= 512 ? 8 : 1;
    TS_REQUIRE(num_tokens <= 65535 * group, "short_conv: %d tokens a step are not supported", num_tokens);
    const dim3 blocks((channels + 255) / 256, (num_tokens + group - 1) / group);
    const unsigned blocks2 = (unsigned)(((long long)num_seqs * channels + 255) / 256);
    if (dtype == TS_F32) {
        short_conv_silu_kernel<float><<<blocks, 256, 0, stream>>>((const float*)x, x_stride, w, seq_of_token, cu_q, slots,
                                                                  state, slot_stride, y, num_tokens, channels, taps, group);
        if (taps > 1)
            short_conv_advance_kernel<float><<<blocks2, 256, 0, stream>>>((const float*)x, x_stride, cu_q, slots, state,
                                                                          slot_stride, num_seqs, channels, taps);
    } else if (dtype == TS_BF16) {
        short_conv_silu_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, x_stride, w, seq_of_token,
                                                                          cu_q, slots, state, slot_stride, y, num_tokens, channels, taps, group);
        if (taps > 1)
            short_conv_advance_kernel<__nv_bfloat16><<<blocks2, 256, 0, stream>>>((const __nv_bfloat16*)x, x_stride, cu_q, slots,
                                                                                  state, slot_stride, num_seqs, channels, taps);
    } else {
        return ts_fail("short_conv: unknown dtype code %d", dtype);
    }
    TS_LAUNCH_CHECK("short_conv");
    return 0;
}
