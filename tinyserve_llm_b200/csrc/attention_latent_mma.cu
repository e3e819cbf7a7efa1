// Attention over a cached latent on bfloat16 tensor cores (mma.sync m16n8k16, float32 accumulation): the
// same computation as ts_latent_attention, for latents of 32 to 512 channels in steps of 32 (64 above 192,
// 128 above 384) and rotated parts of a multiple of 16.
//
// Since all heads of a token read the same cache rows [c | k_rot], the heads are the rows of the products:
// a CTA takes one token and 16 heads, S[16 heads, 64 keys] = Q_abs K^T over rank + rot channels, softmax
// across the keys in float32, O[16 heads, rank] += P C with the same shared-memory tile of keys as the
// second operand (read transposed).  Four warps: each scores 16 of the tile's 64 keys and owns a quarter
// of the output channels; the row maxima go through shared memory so that all warps rescale alike, the
// row sums stay per warp until the end.  Key tiles are copied with cp.async (rows of keys outside the
// window are zero-filled and masked); two CTAs share an SM, one loading while the other computes.
// Two operands enter their product as the sum of two bfloat16 pieces (a second MMA each): the folded query's
// latent part, whose rounding the unfolded form of the attention does not have, and the probabilities; the
// logits then differ from the float32 kernel's no more than that kernel's from the plain model (measured: the
// largest error of a replay fell from 0.5 to 0.3 of its bound, for 15 % of the kernel's time).
// A small step's keys may be split over CTAs exactly as in the FFMA kernel; the partial results have the
// same form and the same kernel merges them.
#include "common.cuh"

constexpr int LM_WARPS = 4, LM_HEADS = 16, LM_KEYS = 64, LM_PAD = 8;

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async_16(void* dst, const void* src, bool valid) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;                      // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(d), "l"(src), "r"(bytes) : "memory");
}

// NT: output n-tiles of 8 channels a warp (rank = 32 NT)
template <int NT>
__global__ void __launch_bounds__(LM_WARPS * 32)
latent_attention_mma_kernel(const float* __restrict__ q_lat, long long ql_token_stride, long long ql_head_stride,
                            const __nv_bfloat16* __restrict__ q, long long q_stride, int q_head_width, int q_rot_offset,
                            const float* __restrict__ freq, const __nv_bfloat16* __restrict__ k_pool, KVGeometry geo,
                            const int* __restrict__ block_table, int table_width, const int* __restrict__ positions,
                            const int* __restrict__ seq_of_token, __nv_bfloat16* __restrict__ out, int heads, int rot,
                            float scale, int window, int split_keys, float* __restrict__ partial) {
    constexpr int RANK = 32 * NT;
    extern __shared__ __align__(16) unsigned char raw[];
    const int width = RANK + rot, pitch = width + LM_PAD;
    const int lpitch = RANK + LM_PAD;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(raw);            // [16][pitch]: the folded queries, rounded
    __nv_bfloat16* Ql = Qs + LM_HEADS * pitch;                            // [16][lpitch]: what rounding left of their latent part
    __nv_bfloat16* Ks = Ql + LM_HEADS * lpitch;                           // [64][pitch]
    __nv_bfloat16* Ps = Ks + LM_KEYS * pitch;                             // [16][64 + pad]
    __nv_bfloat16* Pl = Ps + LM_HEADS * (LM_KEYS + LM_PAD);
    float* red = reinterpret_cast<float*>(Pl + LM_HEADS * (LM_KEYS + LM_PAD));   // [4 warps][16 rows]
    long long* row_base = reinterpret_cast<long long*>(red + LM_WARPS * LM_HEADS);   // [64] element offset of a key's row, -1: none
    const int t = blockIdx.x;
    const int seq = seq_of_token[t];
    if (seq < 0) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h0 = blockIdx.y * LM_HEADS;
    const int pos = positions[t];
    // the folded queries of the 16 heads: [W_uk^T q_flat | rotated q_rot], rounded to bfloat16
    for (int e = tid; e < LM_HEADS * RANK; e += blockDim.x) {
        const int r = e / RANK, d = e % RANK;
        const float x = h0 + r < heads ? q_lat[(long long)t * ql_token_stride + (long long)(h0 + r) * ql_head_stride + d] : 0.f;
        const __nv_bfloat16 hi = __float2bfloat16_rn(x);
        Qs[r * pitch + d] = hi;
        Ql[r * lpitch + d] = __float2bfloat16_rn(x - __bfloat162float(hi));
    }
    const int half = rot / 2;
    for (int e = tid; e < LM_HEADS * half; e += blockDim.x) {
        const int r = e / half, i = e % half;
        float a = 0.f, b = 0.f;
        if (h0 + r < heads) {
            const __nv_bfloat16* qr = q + (long long)t * q_stride + (long long)(h0 + r) * q_head_width + q_rot_offset;
            float sn, cs;
            sincosf((float)pos * freq[i], &sn, &cs);
            const float u = __bfloat162float(qr[i]), v = __bfloat162float(qr[i + half]);
            a = u * cs - v * sn;
            b = v * cs + u * sn;
        }
        Qs[r * pitch + RANK + i] = __float2bfloat16_rn(a);
        Qs[r * pitch + RANK + i + half] = __float2bfloat16_rn(b);
    }
    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[n][c] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};        // rows lane / 4 and lane / 4 + 8
    const int first_key = window > 0 ? max(0, pos - window + 1) : 0;
    const int lo = first_key + (split_keys > 0 ? (int)blockIdx.z * split_keys : 0);
    const int hi = split_keys > 0 ? min(pos, lo + split_keys - 1) : pos;
    const int* table = block_table + (long long)seq * table_width;
    const int chunks = width / 8;
    const int row = lane >> 2, quad = lane & 3;
    for (int j0 = lo; j0 <= hi; j0 += LM_KEYS) {
        const int n = min(LM_KEYS, hi - j0 + 1);
        __syncthreads();                                   // the tile before has been read (first: Qs is written)
        if (tid < LM_KEYS) {
            long long base = -1;
            if (tid < n) {
                const int j = j0 + tid;
                const int page = table[j / geo.page_tokens];
                if (page >= 0 && page < geo.num_pages)
                    base = (long long)page * geo.page_stride + geo.entry_offset + (long long)(j % geo.page_tokens) * width;
            }
            row_base[tid] = base;
        }
        __syncthreads();
        for (int e = tid; e < LM_KEYS * chunks; e += blockDim.x) {
            const int r = e / chunks, c = e % chunks;
            const long long base = row_base[r];
            cp_async_16(Ks + r * pitch + c * 8, k_pool + (base >= 0 ? base : 0) + c * 8, base >= 0);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        // ---- scores of this warp's 16 keys
        float s[2][4];
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int c = 0; c < 4; ++c) s[i][c] = 0.f;
        const int key0 = warp * 16;
        for (int k0 = 0; k0 < width; k0 += 16) {
            unsigned a[4], b[4];
            ldmatrix_x4(a, Qs + (lane & 15) * pitch + k0 + (lane >> 4) * 8);
            ldmatrix_x4(b, Ks + (key0 + ((lane >> 4) << 3) + (lane & 7)) * pitch + k0 + ((lane >> 3) & 1) * 8);
            mma_bf16(s[0], a, b[0], b[1]);
            mma_bf16(s[1], a, b[2], b[3]);
            if (k0 < RANK) {
                // W_uk^T q_flat as the sum of two bfloat16 pieces: folding adds a rounding the unfolded form does not
                // have (many terms that cancel), and this keeps it out of the scores
                ldmatrix_x4(a, Ql + (lane & 15) * lpitch + k0 + (lane >> 4) * 8);
                mma_bf16(s[0], a, b[0], b[1]);
                mma_bf16(s[1], a, b[2], b[3]);
            }
        }
        // thread: rows `row` (c 0, 1) and `row + 8` (c 2, 3); keys key0 + 8 i + 2 quad + {0, 1}
        float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int key = key0 + 8 * i + 2 * quad + (c & 1);
                s[i][c] = key < n && row_base[key] >= 0 ? s[i][c] * scale : -INFINITY;
                tile_max[c >> 1] = fmaxf(tile_max[c >> 1], s[i][c]);
            }
#pragma unroll
        for (int r2 = 0; r2 < 2; ++r2) {
            tile_max[r2] = fmaxf(tile_max[r2], __shfl_xor_sync(0xffffffffu, tile_max[r2], 1));
            tile_max[r2] = fmaxf(tile_max[r2], __shfl_xor_sync(0xffffffffu, tile_max[r2], 2));
        }
        if (quad == 0) {
            red[warp * LM_HEADS + row] = tile_max[0];
            red[warp * LM_HEADS + row + 8] = tile_max[1];
        }
        __syncthreads();
        float corr[2];
#pragma unroll
        for (int r2 = 0; r2 < 2; ++r2) {
            float m_new = m_run[r2];
#pragma unroll
            for (int w = 0; w < LM_WARPS; ++w) m_new = fmaxf(m_new, red[w * LM_HEADS + row + 8 * r2]);
            corr[r2] = m_new == -INFINITY ? 1.f : expf(m_run[r2] - m_new);
            m_run[r2] = m_new;
            l_run[r2] *= corr[r2];
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            float pr[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                pr[c] = s[i][c] == -INFINITY ? 0.f : expf(s[i][c] - m_run[c >> 1]);
                l_run[c >> 1] += pr[c];
            }
            const int col = key0 + 8 * i + 2 * quad;
            const __nv_bfloat162 h01 = __floats2bfloat162_rn(pr[0], pr[1]), h23 = __floats2bfloat162_rn(pr[2], pr[3]);
            *reinterpret_cast<__nv_bfloat162*>(Ps + row * (LM_KEYS + LM_PAD) + col) = h01;
            *reinterpret_cast<__nv_bfloat162*>(Ps + (row + 8) * (LM_KEYS + LM_PAD) + col) = h23;
            *reinterpret_cast<__nv_bfloat162*>(Pl + row * (LM_KEYS + LM_PAD) + col) =
                __floats2bfloat162_rn(pr[0] - __low2float(h01), pr[1] - __high2float(h01));
            *reinterpret_cast<__nv_bfloat162*>(Pl + (row + 8) * (LM_KEYS + LM_PAD) + col) =
                __floats2bfloat162_rn(pr[2] - __low2float(h23), pr[3] - __high2float(h23));
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            o[nt][0] *= corr[0]; o[nt][1] *= corr[0];
            o[nt][2] *= corr[1]; o[nt][3] *= corr[1];
        }
        __syncthreads();                                   // all of P is written
        // ---- this warp's quarter of the output channels: O += P C
        const int ch0 = warp * (RANK / LM_WARPS);
#pragma unroll
        for (int kk = 0; kk < LM_KEYS; kk += 16) {
            unsigned a[4], al[4];
            ldmatrix_x4(a, Ps + (lane & 15) * (LM_KEYS + LM_PAD) + kk + (lane >> 4) * 8);
            ldmatrix_x4(al, Pl + (lane & 15) * (LM_KEYS + LM_PAD) + kk + (lane >> 4) * 8);
#pragma unroll
            for (int nt = 0; nt < NT; nt += 2) {
                // two n-tiles a load; behind an odd last one lie the next warp's channels, the rotated part or the row's
                // padding: read, not used
                unsigned b[4];
                ldmatrix_x4_trans(b, Ks + (kk + ((lane >> 3) & 1) * 8 + (lane & 7)) * pitch + ch0 + nt * 8 + (lane >> 4) * 8);
                mma_bf16(o[nt], a, b[0], b[1]);
                mma_bf16(o[nt], al, b[0], b[1]);
                if (nt + 1 < NT) {
                    mma_bf16(o[nt + 1 < NT ? nt + 1 : nt], a, b[2], b[3]);
                    mma_bf16(o[nt + 1 < NT ? nt + 1 : nt], al, b[2], b[3]);
                }
            }
        }
    }
    // ---- the rows' sums over the four warps, then the output
#pragma unroll
    for (int r2 = 0; r2 < 2; ++r2) {
        l_run[r2] += __shfl_xor_sync(0xffffffffu, l_run[r2], 1);
        l_run[r2] += __shfl_xor_sync(0xffffffffu, l_run[r2], 2);
    }
    __syncthreads();
    if (quad == 0) {
        red[warp * LM_HEADS + row] = l_run[0];
        red[warp * LM_HEADS + row + 8] = l_run[1];
    }
    __syncthreads();
    const int ch0 = warp * (RANK / LM_WARPS);
#pragma unroll
    for (int r2 = 0; r2 < 2; ++r2) {
        const int h = h0 + row + 8 * r2;
        if (h >= heads) continue;
        float l = 0.f;
#pragma unroll
        for (int w = 0; w < LM_WARPS; ++w) l += red[w * LM_HEADS + row + 8 * r2];
        if (split_keys > 0) {
            float* dst = partial + (((long long)t * heads + h) * gridDim.z + blockIdx.z) * (RANK + 2);
            if (warp == 0 && quad == 0) { dst[0] = m_run[r2]; dst[1] = l; }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                dst[2 + ch0 + nt * 8 + 2 * quad] = o[nt][2 * r2];
                dst[2 + ch0 + nt * 8 + 2 * quad + 1] = o[nt][2 * r2 + 1];
            }
        } else {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            __nv_bfloat16* dst = out + ((long long)t * heads + h) * RANK;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
                *reinterpret_cast<__nv_bfloat162*>(dst + ch0 + nt * 8 + 2 * quad) =
                    __floats2bfloat162_rn(o[nt][2 * r2] * inv, o[nt][2 * r2 + 1] * inv);
        }
    }
}

static bool g_latent_mma = true;

TS_API void ts_set_latent_mma(int enabled) { g_latent_mma = enabled != 0; }

bool ts_latent_mma_supported(int rank, int rot) {
    if (!g_latent_mma || rank % 32 || rot % 16 || rot < 0) return false;
    const int nt = rank / 32;
    return nt == 1 || nt == 2 || nt == 3 || nt == 4 || nt == 5 || nt == 6 || nt == 8 || nt == 10 || nt == 12 || nt == 16;
}

int ts_latent_attention_mma_launch(const float* q_lat, long long ql_t, long long ql_h, const void* q, long long q_stride,
                                   int q_head_width, int q_rot_offset, const float* freq, const void* k_pool,
                                   KVGeometry geo, const int* block_table, int table_width, const int* positions,
                                   const int* seq_of_token, void* out, int num_tokens, int heads, int rank, int rot,
                                   float scale, int window, int split_keys, int splits, float* partial,
                                   cudaStream_t stream) {
    const int width = rank + rot, pitch = width + LM_PAD;
    const size_t smem = (size_t)(LM_HEADS + LM_KEYS) * pitch * 2 + (size_t)LM_HEADS * (rank + LM_PAD) * 2 +
                        (size_t)2 * LM_HEADS * (LM_KEYS + LM_PAD) * 2 +
                        (size_t)LM_WARPS * LM_HEADS * 4 + (size_t)LM_KEYS * 8;
    dim3 grid(num_tokens, (heads + LM_HEADS - 1) / LM_HEADS, split_keys > 0 ? splits : 1);
#define TS_LATENT_MMA(NT)                                                                                              \
    do {                                                                                                               \
        if (smem > 48 * 1024)                                                                                          \
            cudaFuncSetAttribute(latent_attention_mma_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        latent_attention_mma_kernel<NT><<<grid, LM_WARPS * 32, smem, stream>>>(                                        \
            q_lat, ql_t, ql_h, (const __nv_bfloat16*)q, q_stride, q_head_width, q_rot_offset, freq,                    \
            (const __nv_bfloat16*)k_pool, geo, block_table, table_width, positions, seq_of_token, (__nv_bfloat16*)out, \
            heads, rot, scale, window, split_keys, partial);                                                           \
    } while (0)
    switch (rank / 32) {
        case 1: TS_LATENT_MMA(1); break;
        case 2: TS_LATENT_MMA(2); break;
        case 3: TS_LATENT_MMA(3); break;
        case 4: TS_LATENT_MMA(4); break;
        case 5: TS_LATENT_MMA(5); break;
        case 6: TS_LATENT_MMA(6); break;
        case 10: TS_LATENT_MMA(10); break;
        case 8: TS_LATENT_MMA(8); break;
        case 12: TS_LATENT_MMA(12); break;
        case 16: TS_LATENT_MMA(16); break;
        default: return ts_fail("latent_attention (mma): a latent of %d channels is not supported", rank);
    }
#undef TS_LATENT_MMA
    TS_LAUNCH_CHECK("latent_attention (mma)");
    return 0;
}
