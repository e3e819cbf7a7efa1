// Linear attention as a recurrence with a decayed matrix state per request and head:
//
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T        S: [key channels, value channels], float32
//   o_t = S_t^T q_t
//
// with a_t either one constant per head (retention) or one value per key channel computed from a
// projection's output z:  a = sigmoid(z + bias)^(1/tau), taken as exp(log_sigmoid(z + bias) / tau)
// (gated linear attention).  q and k may be rotated (rotate-half over the first `rot_dims` channels
// of a head, angle = position * freq[i]) and scaled on their way in.  Everything from the loaded
// projections on is float32: rotation, decays, the state, the sums.
//
// One kernel serves prompts, portions of prompts and single decoded tokens: a CTA owns one request,
// one head and 16 value channels (8 for the delta rule), reads the state from the request's slot, walks over the request's
// tokens of this step in order and writes the state back.  The arithmetic of a token does not depend
// on where the step was cut or on what else is in the batch.  A first kernel computes what enters
// the recurrence (rotated and scaled q and k, the decays) once per token, head and channel; the scan
// stages 16 tokens of it at a time, fetched one tile ahead.  Inside a tile no thread waits for
// another: thread (r, j) holds a run of rows of column j of S (read from the staged tile four
// channels a load) and leaves its share of o_t[j] in shared memory, and the sixteen shares are added
// up in a fixed order after the tile.
//
// A second kernel norms each head's o over the value channels (with or without a weight),
// multiplies by silu(gate) or sigmoid(gate) and rounds to the activation dtype for the output projection.
//
// The scan also runs the delta rule (`beta` given):
//   S <- diag(a_t) S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t
// where the read S^T k_t feeds back into the state, so the sixteen threads that share a column of S
// are lanes of one warp and add up their shares with shuffles, token by token.
// A value column past `v_cols` is the constant 1: with it the state carries the sum of the (decayed)
// keys beside the matrix, and o's extra column is that sum's product with q (the normaliser of a
// matrix memory with exponential gates).  The inputs of these variants are prepared by kernels of
// their own, further down.
#include "common.cuh"

constexpr int LR_ROWGROUPS = 16;    // thread (r, j) holds rows r * MAXM .. r * MAXM + MAXM - 1 of column j of the state
constexpr int LR_TILE = 16;         // tokens staged at a time
static_assert(LR_TILE == LR_ROWGROUPS, "a thread stages one value of v a tile: tokens x columns = row groups x columns");

__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// What enters the recurrence, computed once per token, head and key channel (the scan's CTAs of one head all read it):
// prepared[0] = rotated, scaled q; prepared[1] = rotated, scaled k; prepared[2] = the decay a.  Each [tokens, heads * dim].
template <typename T>
__global__ void recurrence_prepare_kernel(const T* __restrict__ q, const T* __restrict__ k, long long q_stride,
                                          long long k_stride, const float* __restrict__ z, long long z_stride,
                                          const float* __restrict__ bias, const float* __restrict__ head_decay,
                                          float inv_tau, float q_scale, float k_scale, const float* __restrict__ freq,
                                          int rot_dims, const int* __restrict__ positions, float* __restrict__ prepared,
                                          long long total, int heads, int dim) {
    const int width = heads * dim, half = rot_dims / 2;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const long long t = e / width;
        const int c = (int)(e % width), h = c / dim, i = c % dim;
        const T* qr = q + t * q_stride + (long long)h * dim;
        const T* kr = k + t * k_stride + (long long)h * dim;
        float qv = to_float<T>(qr[i]), kv = to_float<T>(kr[i]);
        if (freq && i < rot_dims) {
            const int f = i < half ? i : i - half, other = i < half ? i + half : i - half;
            float sn, cs;
            sincosf((float)positions[t] * freq[f], &sn, &cs);
            const float qo = to_float<T>(qr[other]), ko = to_float<T>(kr[other]);
            // first half: u cos - v sin; second half: v cos + u sin
            qv = i < half ? qv * cs - qo * sn : qv * cs + qo * sn;
            kv = i < half ? kv * cs - ko * sn : kv * cs + ko * sn;
        }
        float a = head_decay ? head_decay[h] : 1.f;
        if (z) a = expf(log_sigmoid(z[t * z_stride + c] + (bias ? bias[c] : 0.f)) * inv_tau);
        prepared[e] = qv * q_scale;
        prepared[total + e] = kv * k_scale;
        prepared[2 * total + e] = a;
    }
}

struct RecurrenceArgs {
    const float* prepared; long long total;           // [3][tokens, heads * dim]: q, k, decay as they enter the recurrence
    const void* v; long long v_stride;                // elements between tokens; a head's values start at h * v_cols
    int v_cols;                                       // value columns read from v; columns from here to vdim are 1
    const float* beta;                                // [tokens, heads]: the delta rule's step size (null: plain recurrence)
    const int* cu_q; const int* slots;
    float* state; long long slot_stride;              // floats between slots; a slot holds [heads, dim, vdim]
    float* out;                                       // [tokens, heads * vdim] float32
    int heads, dim, vdim;
};

// COLS: value channels of a CTA (16; the delta rule, whose tokens are a chain of dependent steps, runs 8 a CTA so that
// a prompt alone spreads over twice the SMs)
template <typename T, int MAXM, bool DELTA, int COLS>
__global__ void __launch_bounds__(LR_ROWGROUPS * COLS)
linear_recurrence_kernel(RecurrenceArgs p) {
    // staged rows are padded with zeros to LR_ROWGROUPS * MAXM channels: the inner loop needs no bound and reads
    // four channels a load
    constexpr int PITCH = LR_ROWGROUPS * MAXM;
    extern __shared__ __align__(16) float smem[];
    const int dim = p.dim, vdim = p.vdim;
    float* q_s = smem;                                   // [LR_TILE][PITCH]
    float* k_s = q_s + LR_TILE * PITCH;
    float* a_s = k_s + LR_TILE * PITCH;
    float* v_s = a_s + LR_TILE * PITCH;                  // [LR_TILE][COLS]
    float* part = v_s + LR_TILE * COLS;               // [LR_TILE][LR_ROWGROUPS][COLS]
    float* b_s = part + LR_TILE * LR_ROWGROUPS * COLS; // [LR_TILE] (delta rule)
    const int seq = blockIdx.z, h = blockIdx.y, j0 = blockIdx.x * COLS;
    const int slot = p.slots[seq];
    const int begin = p.cu_q[seq], end = p.cu_q[seq + 1];
    if (slot < 0 || end <= begin) return;                // a padding request, or one that feeds nothing
    // plain: the threads of a row group are neighbours (their loads of a state row coalesce); delta rule: the
    // sixteen row groups of a column are the lanes of half a warp
    const int r = DELTA ? threadIdx.x % LR_ROWGROUPS : threadIdx.x / COLS;
    const int jj = DELTA ? threadIdx.x / LR_ROWGROUPS : threadIdx.x % COLS, j = j0 + jj;
    const bool live = j < vdim;
    float* st = p.state + (long long)slot * p.slot_stride + (long long)h * dim * vdim;
    // Which rows of its column a thread holds.  Plain: a run of MAXM rows.  Delta rule: four rows out of every 64, so that
    // the sixteen lanes of a column read one contiguous stretch of a staged row with each 16-byte load (a run a lane
    // would put the lanes' loads 4 * MAXM bytes apart: two to four passes through shared memory a load)
    auto row_of = [&](int m) { return DELTA ? (m >> 2) * (4 * LR_ROWGROUPS) + 4 * r + (m & 3) : r * MAXM + m; };
    const int first = DELTA ? 4 * r : r * MAXM;           // floats from a staged row's start to this thread's first 16 bytes
    constexpr int STEP4 = DELTA ? LR_ROWGROUPS : 1;       // float4s between a thread's consecutive 16-byte loads
    float S[MAXM];
#pragma unroll
    for (int m = 0; m < MAXM; ++m) {
        const int i = row_of(m);
        S[m] = (live && i < dim) ? st[(long long)i * vdim + j] : 0.f;
    }
    const T* v = (const T*)p.v;
    const long long row_width = (long long)p.heads * dim;
    // What a tile needs from global memory is asked for one tile ahead and held in registers while the tile
    // before it is worked on.
    constexpr int ROUNDS = LR_TILE * PITCH / (LR_ROWGROUPS * COLS);
    float raw_q[ROUNDS], raw_k[ROUNDS], raw_a[ROUNDS];
    T raw_v;                                             // as loaded: converting would wait for the load
    float raw_b = 0.f;
    auto fetch = [&](int t0, int n) {
#pragma unroll
        for (int round = 0; round < ROUNDS; ++round) {
            const int e = round * (LR_ROWGROUPS * COLS) + threadIdx.x;
            const int tt = e / PITCH, i = e % PITCH;
            raw_q[round] = raw_k[round] = raw_a[round] = 0.f;
            if (tt < n && i < dim) {
                const long long at = (long long)(t0 + tt) * row_width + (long long)h * dim + i;
                raw_q[round] = p.prepared[at];
                raw_k[round] = p.prepared[p.total + at];
                raw_a[round] = p.prepared[2 * p.total + at];
            }
        }
        const int tt = threadIdx.x / COLS, c = threadIdx.x % COLS;       // LR_TILE * COLS = one value a thread
        raw_v = from_float<T>(j0 + c >= p.v_cols && j0 + c < vdim ? 1.f : 0.f);
        if (tt < n && j0 + c < p.v_cols) raw_v = v[(long long)(t0 + tt) * p.v_stride + (long long)h * p.v_cols + j0 + c];
        if (DELTA && threadIdx.x < LR_TILE) raw_b = threadIdx.x < n ? p.beta[(long long)(t0 + threadIdx.x) * p.heads + h] : 0.f;
    };
    fetch(begin, min(LR_TILE, end - begin));
    for (int t0 = begin; t0 < end; t0 += LR_TILE) {
        const int n = min(LR_TILE, end - t0);
        __syncthreads();                                 // the tile before has been read
#pragma unroll
        for (int round = 0; round < ROUNDS; ++round) {
            const int e = round * (LR_ROWGROUPS * COLS) + threadIdx.x;
            q_s[e] = raw_q[round];
            k_s[e] = raw_k[round];
            a_s[e] = raw_a[round];
        }
        v_s[threadIdx.x] = to_float<T>(raw_v);
        if (DELTA && threadIdx.x < LR_TILE) b_s[threadIdx.x] = raw_b;
        if (t0 + LR_TILE < end) fetch(t0 + LR_TILE, min(LR_TILE, end - t0 - LR_TILE));   // under way during this tile's work
        __syncthreads();
        if (DELTA) {
            // The chain from one token's state to the next's is decay, S^T k, four shuffles, the correction.  What a
            // token needs from shared memory is loaded one token ahead, so that the chain waits for nothing else; its
            // sums are kept in four pieces so that no piece waits for more than MAXM / 4 products.
            float4 kc[MAXM / 4], ac4[MAXM / 4], qc[MAXM / 4];
            float vc, bc;
            auto load_token = [&](int tt, float4 (&k4)[MAXM / 4], float4 (&a4)[MAXM / 4], float4 (&q4)[MAXM / 4], float& vv,
                                  float& bb) {
                const float4* qt = reinterpret_cast<const float4*>(q_s + tt * PITCH + first);
                const float4* kt = reinterpret_cast<const float4*>(k_s + tt * PITCH + first);
                const float4* at = reinterpret_cast<const float4*>(a_s + tt * PITCH + first);
#pragma unroll
                for (int m4 = 0; m4 < MAXM / 4; ++m4) { k4[m4] = kt[m4 * STEP4]; a4[m4] = at[m4 * STEP4]; q4[m4] = qt[m4 * STEP4]; }
                vv = v_s[tt * COLS + jj];
                bb = b_s[tt];
            };
            load_token(0, kc, ac4, qc, vc, bc);
            for (int tt = 0; tt < n; ++tt) {
                float4 kn[MAXM / 4], an[MAXM / 4], qn[MAXM / 4];
                float vn, bn;
                load_token(min(tt + 1, LR_TILE - 1), kn, an, qn, vn, bn);      // the tile's last row again: not used
                float rd[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int m4 = 0; m4 < MAXM / 4; ++m4) {
                    const float kk[4] = {kc[m4].x, kc[m4].y, kc[m4].z, kc[m4].w};
                    const float aa[4] = {ac4[m4].x, ac4[m4].y, ac4[m4].z, ac4[m4].w};
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int m = 4 * m4 + c;
                        S[m] *= aa[c];
                        rd[c] = fmaf(S[m], kk[c], rd[c]);
                    }
                }
                float read = (rd[0] + rd[1]) + (rd[2] + rd[3]);
#pragma unroll
                for (int o = LR_ROWGROUPS / 2; o > 0; o >>= 1) read += __shfl_xor_sync(0xffffffffu, read, o);
                const float u = bc * (vc - read);
                float ac[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int m4 = 0; m4 < MAXM / 4; ++m4) {
                    const float kk[4] = {kc[m4].x, kc[m4].y, kc[m4].z, kc[m4].w};
                    const float qq[4] = {qc[m4].x, qc[m4].y, qc[m4].z, qc[m4].w};
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int m = 4 * m4 + c;
                        S[m] = fmaf(kk[c], u, S[m]);
                        ac[c] = fmaf(S[m], qq[c], ac[c]);
                    }
                }
                part[(tt * LR_ROWGROUPS + r) * COLS + jj] = (ac[0] + ac[1]) + (ac[2] + ac[3]);
#pragma unroll
                for (int m4 = 0; m4 < MAXM / 4; ++m4) { kc[m4] = kn[m4]; ac4[m4] = an[m4]; qc[m4] = qn[m4]; }
                vc = vn;
                bc = bn;
            }
        } else {
            // no thread waits for another here; a token's staged inputs are loaded one token ahead of their use
            float4 kc[MAXM / 4], ac4[MAXM / 4], qc[MAXM / 4];
            float vc;
            auto load_token = [&](int tt, float4 (&k4)[MAXM / 4], float4 (&a4)[MAXM / 4], float4 (&q4)[MAXM / 4], float& vv) {
                const float4* qt = reinterpret_cast<const float4*>(q_s + tt * PITCH + first);
                const float4* kt = reinterpret_cast<const float4*>(k_s + tt * PITCH + first);
                const float4* at = reinterpret_cast<const float4*>(a_s + tt * PITCH + first);
#pragma unroll
                for (int m4 = 0; m4 < MAXM / 4; ++m4) { k4[m4] = kt[m4]; a4[m4] = at[m4]; q4[m4] = qt[m4]; }
                vv = v_s[tt * COLS + jj];
            };
            load_token(0, kc, ac4, qc, vc);
            for (int tt = 0; tt < n; ++tt) {
                float4 kn[MAXM / 4], an[MAXM / 4], qn[MAXM / 4];
                float vn;
                load_token(min(tt + 1, LR_TILE - 1), kn, an, qn, vn);          // the tile's last row again: not used
                float acc = 0.f;
#pragma unroll
                for (int m4 = 0; m4 < MAXM / 4; ++m4) {
                    const float qq[4] = {qc[m4].x, qc[m4].y, qc[m4].z, qc[m4].w}, kk[4] = {kc[m4].x, kc[m4].y, kc[m4].z, kc[m4].w};
                    const float aa[4] = {ac4[m4].x, ac4[m4].y, ac4[m4].z, ac4[m4].w};
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int m = 4 * m4 + c;
                        S[m] = fmaf(aa[c], S[m], kk[c] * vc);
                        acc = fmaf(S[m], qq[c], acc);
                    }
                }
                part[(tt * LR_ROWGROUPS + r) * COLS + jj] = acc;
#pragma unroll
                for (int m4 = 0; m4 < MAXM / 4; ++m4) { kc[m4] = kn[m4]; ac4[m4] = an[m4]; qc[m4] = qn[m4]; }
                vc = vn;
            }
        }
        __syncthreads();
        for (int e = threadIdx.x; e < n * COLS; e += blockDim.x) {
            const int tt = e / COLS, c = e % COLS;
            if (j0 + c >= vdim) continue;
            float o = 0.f;
#pragma unroll
            for (int g = 0; g < LR_ROWGROUPS; ++g) o += part[(tt * LR_ROWGROUPS + g) * COLS + c];
            p.out[(long long)(t0 + tt) * p.heads * vdim + (long long)h * vdim + j0 + c] = o;
        }
    }
#pragma unroll
    for (int m = 0; m < MAXM; ++m) {
        const int i = row_of(m);
        if (live && i < dim) st[(long long)i * vdim + j] = S[m];
    }
}

template <typename T>
static int launch_recurrence(const RecurrenceArgs& p, int num_seqs, cudaStream_t stream) {
#define TS_RECURRENCE(MAXM, DELTA, COLS)                                                                           \
    do {                                                                                                           \
        const dim3 grid((p.vdim + COLS - 1) / COLS, p.heads, num_seqs);                                            \
        const size_t smem = (size_t)(3 * LR_TILE * LR_ROWGROUPS * MAXM + LR_TILE * COLS +                          \
                                     LR_TILE * LR_ROWGROUPS * COLS + LR_TILE) * sizeof(float);                     \
        if (smem > 48 * 1024)                                                                                      \
            cudaFuncSetAttribute(linear_recurrence_kernel<T, MAXM, DELTA, COLS>,                                   \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                          \
        linear_recurrence_kernel<T, MAXM, DELTA, COLS><<<grid, LR_ROWGROUPS * COLS, smem, stream>>>(p);            \
    } while (0)
    if (p.beta) {
        if (p.dim <= 4 * LR_ROWGROUPS) TS_RECURRENCE(4, true, 8);
        else if (p.dim <= 8 * LR_ROWGROUPS) TS_RECURRENCE(8, true, 8);
        else TS_RECURRENCE(16, true, 16);
    } else {
        if (p.dim <= 4 * LR_ROWGROUPS) TS_RECURRENCE(4, false, 16);
        else if (p.dim <= 8 * LR_ROWGROUPS) TS_RECURRENCE(8, false, 16);
        else TS_RECURRENCE(16, false, 16);
    }
#undef TS_RECURRENCE
    TS_LAUNCH_CHECK("linear_recurrence");
    return 0;
}

// The scan alone, from inputs a kernel of the caller's prepared: prepared [3][tokens, heads * dim] float32
// (q, k and the decay as they enter the recurrence), v [tokens, heads * v_cols] in float32 or the activation
// dtype, beta [tokens, heads] or null.  A slot holds [heads, dim, vdim] floats.
TS_API int ts_recurrence_scan(const float* prepared, const void* v, long long v_stride, int v_cols, int v_dtype,
                              const float* beta, const int* cu_q, const int* slots, int num_seqs, float* state,
                              long long slot_stride, float* out, int heads, int dim, int vdim, int num_tokens,
                              cudaStream_t stream) {
    TS_REQUIRE(heads > 0 && dim > 0 && vdim > 0 && num_seqs >= 0 && num_tokens >= 0, "recurrence_scan: bad sizes");
    TS_REQUIRE(dim <= 16 * LR_ROWGROUPS, "recurrence_scan: %d key channels a head are not supported (up to %d)", dim,
               16 * LR_ROWGROUPS);
    TS_REQUIRE(v_cols >= 0 && v_cols <= vdim, "recurrence_scan: %d of %d value columns", v_cols, vdim);
    TS_REQUIRE(slot_stride >= (long long)heads * dim * vdim, "recurrence_scan: a state slot is too small");
    TS_REQUIRE(num_seqs <= 65535 && heads <= 65535, "recurrence_scan: grid too large");
    if (num_seqs == 0 || num_tokens == 0) return 0;
    const long long total = (long long)num_tokens * heads * dim;
    RecurrenceArgs p{prepared, total, v, v_stride, v_cols, beta, cu_q, slots, state, slot_stride, out, heads, dim, vdim};
    if (v_dtype == TS_F32) return launch_recurrence<float>(p, num_seqs, stream);
    if (v_dtype == TS_BF16) return launch_recurrence<__nv_bfloat16>(p, num_seqs, stream);
    return ts_fail("recurrence_scan: unknown dtype code %d", v_dtype);
}

TS_API int ts_linear_recurrence(const void* q, const void* k, const void* v, long long q_stride, long long k_stride,
                                long long v_stride, const float* z, long long z_stride, const float* bias,
                                const float* head_decay, float inv_tau, float q_scale, float k_scale, const float* freq,
                                int rot_dims, const int* positions, const int* cu_q, const int* slots, int num_seqs,
                                float* state, long long slot_stride, float* out, int heads, int dim, int vdim,
                                int num_tokens, float* prepared, int dtype, cudaStream_t stream) {
    TS_REQUIRE(heads > 0 && dim > 0 && vdim > 0 && num_seqs >= 0 && num_tokens >= 0, "linear_recurrence: bad sizes");
    TS_REQUIRE(dim <= 16 * LR_ROWGROUPS, "linear_recurrence: %d key channels a head are not supported (up to %d)", dim,
               16 * LR_ROWGROUPS);
    TS_REQUIRE(rot_dims >= 0 && rot_dims <= dim && rot_dims % 2 == 0, "linear_recurrence: rotation over %d of %d channels",
               rot_dims, dim);
    TS_REQUIRE((z != nullptr) != (head_decay != nullptr), "linear_recurrence: either decay logits or one decay per head");
    TS_REQUIRE(slot_stride >= (long long)heads * dim * vdim, "linear_recurrence: a state slot is too small");
    TS_REQUIRE(num_seqs <= 65535 && heads <= 65535, "linear_recurrence: grid too large");
    TS_REQUIRE(prepared != nullptr || num_tokens == 0, "linear_recurrence: no room for the prepared inputs");
    if (num_seqs == 0 || num_tokens == 0) return 0;
    const long long total = (long long)num_tokens * heads * dim;
    const unsigned blocks = (unsigned)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    const float* fr = rot_dims > 0 ? freq : nullptr;
    if (dtype == TS_F32)
        recurrence_prepare_kernel<float><<<blocks, 256, 0, stream>>>((const float*)q, (const float*)k, q_stride, k_stride, z,
            z_stride, bias, head_decay, inv_tau, q_scale, k_scale, fr, rot_dims, positions, prepared, total, heads, dim);
    else if (dtype == TS_BF16)
        recurrence_prepare_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k,
            q_stride, k_stride, z, z_stride, bias, head_decay, inv_tau, q_scale, k_scale, fr, rot_dims, positions, prepared,
            total, heads, dim);
    else
        return ts_fail("linear_recurrence: unknown dtype code %d", dtype);
    TS_LAUNCH_CHECK("linear_recurrence (prepare)");
    RecurrenceArgs p{prepared, total, v, v_stride, vdim, nullptr, cu_q, slots, state, slot_stride, out, heads, dim, vdim};
    if (dtype == TS_F32) return launch_recurrence<float>(p, num_seqs, stream);
    return launch_recurrence<__nv_bfloat16>(p, num_seqs, stream);
}

// out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * weight * act(gate[t, h, :]) * scale; one warp a
// (token, head).  `gate_kind` 0: silu, 1: sigmoid.  The weight is shared by the heads (`weight_stride` 0) or one
// stretch a head (`weight_stride` = vdim).  A head of o is `o_head` floats apart from the next (vdim, or more where
// o carries extra columns).  With `log_max` ([tokens, heads]) the head is first divided by
// max(|o[t, h, vdim]|, exp(-log_max[t, h])) + 1e-6: the normaliser of a matrix memory with exponential gates, whose
// product with q the scan left in column vdim.  The result may be a column stretch of a wider tensor (`out_stride`).
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, int o_head, const T* __restrict__ gate,
                                      long long gate_stride, const float* __restrict__ weight, int weight_stride,
                                      const float* __restrict__ log_max, T* __restrict__ out, long long out_stride,
                                      long long items, int heads, int vdim, float eps, int gate_kind, float scale) {
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= items) return;
    const int lane = threadIdx.x & 31;
    const long long t = item / heads;
    const int h = (int)(item % heads);
    const float* orow = o + item * o_head;
    float pre = 1.f;
    if (log_max) pre = 1.f / (fmaxf(fabsf(orow[vdim]), expf(-log_max[item])) + 1e-6f);
    float acc = 0.f;
    for (int j = lane; j < vdim; j += 32) acc += (orow[j] * pre) * (orow[j] * pre);
    const float inv = 1.f / sqrtf(warp_sum(acc) / (float)vdim + eps);
    const T* g = gate + t * gate_stride + (long long)h * vdim;
    T* dst = out + t * out_stride + (long long)h * vdim;
    const float* w = weight ? weight + (long long)h * weight_stride : nullptr;
    for (int j = lane; j < vdim; j += 32) {
        const float x = to_float<T>(g[j]);
        const float sig = 1.f / (1.f + expf(-x));
        const float act = gate_kind == 1 ? sig : x * sig;
        dst[j] = from_float<T>(orow[j] * pre * inv * (w ? w[j] : 1.f) * act * scale);
    }
}

TS_API int ts_head_norm_gate(const float* o, int o_head, const void* gate, long long gate_stride, const float* weight,
                             int weight_stride, const float* log_max, void* out, long long out_stride, int num_tokens,
                             int heads, int vdim, float eps, int gate_kind, float scale, int dtype, cudaStream_t stream) {
    TS_REQUIRE(num_tokens >= 0 && heads > 0 && vdim > 0 && o_head >= vdim, "head_norm_gate: bad sizes");
    TS_REQUIRE(!log_max || o_head > vdim, "head_norm_gate: the normaliser's column is missing");
    if (num_tokens == 0) return 0;
    const long long items = (long long)num_tokens * heads;
    const unsigned blocks = (unsigned)((items + 3) / 4);
    if (dtype == TS_F32)
        head_norm_gate_kernel<float><<<blocks, 128, 0, stream>>>(o, o_head, (const float*)gate, gate_stride, weight,
            weight_stride, log_max, (float*)out, out_stride, items, heads, vdim, eps, gate_kind, scale);
    else if (dtype == TS_BF16)
        head_norm_gate_kernel<__nv_bfloat16><<<blocks, 128, 0, stream>>>(o, o_head, (const __nv_bfloat16*)gate, gate_stride,
            weight, weight_stride, log_max, (__nv_bfloat16*)out, out_stride, items, heads, vdim, eps, gate_kind, scale);
    else
        return ts_fail("head_norm_gate: unknown dtype code %d", dtype);
    TS_LAUNCH_CHECK("head_norm_gate");
    return 0;
}
