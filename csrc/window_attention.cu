// Attention over the KV cache with a sliding window, kept first tokens ("sinks") and a linear distance bias, for
// per-head query/key size D and value size Dv that need not be equal or a power of two; bf16 or fp32 activations.
//
//   visible(i, j) = j <= i and (window <= 0 or i - j < window or j < keep_first)
//   score(i, j)   = scale * <q_i, k_j> - slope_h * (i - j)            (slopes == NULL: no bias)
//
// Three kernels:
//   qk_norm_cache_write   rows of the fused projection output -> unit-RMS q (written out) and unit-RMS k + v written
//                         into the cache at (line, position); statistics in fp32
//   window_attn_prefill   a tile of 16 queries of one head per CTA, keys and values streamed from the cache in tiles of
//                         32 rows, key tiles that no query of the tile can see are skipped, online softmax in fp32
//   window_attn_decode    one new token per row: one CTA per (row, key/value head), the warps split the visible keys
//                         (kept first tokens, then the window), every warp keeps an online-softmax state for the query
//                         heads of the group, merged through shared memory
// The cache is contiguous [lines, G, S, D] or paged [pages, G, page, D] with a block table [lines, cols].
#include "common.cuh"

namespace {

struct CacheAddr {
    long long stride_line, stride_head;   // elements
    const int* block_table;
    int page_size, table_cols, row_dim;
    __device__ __forceinline__ long long row(int line, int g, int pos) const {
        if (block_table != nullptr) {
            const int page = block_table[(long long)line * table_cols + pos / page_size];
            return (long long)page * stride_line + (long long)g * stride_head + (long long)(pos % page_size) * row_dim;
        }
        return (long long)line * stride_line + (long long)g * stride_head + (long long)pos * row_dim;
    }
};

__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const bf16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// ---------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void qk_norm_cache_write_kernel(const T* __restrict__ qkv, long long ld, T* __restrict__ q_out,
                                           T* __restrict__ cache_k, T* __restrict__ cache_v, CacheAddr ka, CacheAddr va,
                                           const int* __restrict__ q_start, const int* __restrict__ n_new,
                                           const int* __restrict__ seq_ids, long long units, int Tn, int H, int G, int D,
                                           int Dv, int has_kv, int normalize, float eps, int max_pos) {
    const int lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= units) return;
    const int per_row = H + (has_kv ? 2 * G : 0);
    const long long n = unit / per_row;
    const int hd = (int)(unit % per_row);
    const int b = (int)(n / Tn), t = (int)(n % Tn);
    const T* src;
    int dim;
    if (hd < H) {
        src = qkv + n * ld + (long long)hd * D;
        dim = D;
    } else if (hd < H + G) {
        src = qkv + n * ld + (long long)H * D + (long long)(hd - H) * D;
        dim = D;
    } else {
        src = qkv + n * ld + (long long)(H + G) * D + (long long)(hd - H - G) * Dv;
        dim = Dv;
    }
    T* dst;
    if (hd < H) {
        dst = q_out + (n * H + hd) * D;
    } else {
        const bool valid = n_new == nullptr || t < n_new[b];
        const int pos = q_start[b] + t;
        if (!valid || pos >= max_pos || pos < 0) return;
        const int line = seq_ids != nullptr ? seq_ids[b] : b;
        dst = hd < H + G ? cache_k + ka.row(line, hd - H, pos) : cache_v + va.row(line, hd - H - G, pos);
    }
    float r = 1.f;
    if (hd < H + G && normalize) {
        float ss = 0.f;
        for (int i = lane; i < dim; i += 32) {
            const float v = ldf(src + i);
            ss += v * v;
        }
        ss = warp_sum(ss);
        r = 1.f / sqrtf(ss / (float)dim + eps);
    }
    for (int i = lane; i < dim; i += 32) stf(dst + i, ldf(src + i) * r);
}

// ---------------------------------------------------------------------------------------------------------------------
constexpr int BQ = 16, BK = 32, PF_THREADS = 128, MAXC = 32;   // MAXC * 8 = largest value size

template <typename T>
__global__ void __launch_bounds__(PF_THREADS)
window_attn_prefill_kernel(const T* __restrict__ q, const T* __restrict__ cache_k, const T* __restrict__ cache_v,
                           CacheAddr ka, CacheAddr va, T* __restrict__ out, const int* __restrict__ q_start,
                           const int* __restrict__ n_new, const int* __restrict__ seq_ids,
                           const float* __restrict__ slopes, int Tn, int H, int G, int D, int Dv, float scale, int window,
                           int keep_first) {
    extern __shared__ float smem[];
    float* Qs = smem;                       // [BQ][D]
    float* Ks = Qs + BQ * D;                // [BK][D + 1]
    float* Vs = Ks + BK * (D + 1);          // [BK][Dv]
    float* Ps = Vs + BK * Dv;               // [BQ][BK]
    __shared__ long long koff[BK], voff[BK];

    const int tid = threadIdx.x;
    const int q0 = blockIdx.x * BQ, h = blockIdx.y, b = blockIdx.z;
    const int g = h / (H / G);
    const int nb = n_new != nullptr ? min(n_new[b], Tn) : Tn;
    const int qi = tid >> 3, sub = tid & 7;
    const int nc = (Dv + 7) >> 3;
    T* orow = out + (((long long)b * Tn + q0 + qi) * H + h) * Dv;
    if (q0 >= nb) {                          // a tile of padding rows: defined output, no work
        if (q0 + qi < Tn)
            for (int m = 0; m < nc; ++m) {
                const int c = sub + 8 * m;
                if (c < Dv) stf(orow + c, 0.f);
            }
        return;
    }
    const int start = q_start[b];
    const int line = seq_ids != nullptr ? seq_ids[b] : b;
    const int p_lo = start + q0;
    const int p_hi = start + min(q0 + BQ, nb) - 1;
    const float slope = slopes != nullptr ? slopes[h] : 0.f;

    for (int idx = tid; idx < BQ * D; idx += PF_THREADS) {
        const int r = idx / D, c = idx - r * D;
        Qs[idx] = (q0 + r < nb) ? ldf(q + (((long long)b * Tn + q0 + r) * H + h) * D + c) * scale : 0.f;
    }
    const int p_i = start + q0 + qi;
    const bool row_ok = q0 + qi < nb;
    float m_i = -INFINITY, l_i = 0.f;
    float acc[MAXC];
#pragma unroll
    for (int m = 0; m < MAXC; ++m) acc[m] = 0.f;

    const int last_tile = p_hi / BK;
    for (int kt = 0; kt <= last_tile; ++kt) {
        const int k0 = kt * BK;
        if (window > 0 && k0 >= keep_first && k0 + BK - 1 <= p_lo - window) continue;   // nobody in the tile sees it
        __syncthreads();                     // previous tile fully consumed (and Qs written, first time round)
        if (tid < BK) {
            const int pos = k0 + tid;
            koff[tid] = pos <= p_hi ? ka.row(line, g, pos) : -1;
            voff[tid] = pos <= p_hi ? va.row(line, g, pos) : -1;
        }
        __syncthreads();
        for (int idx = tid; idx < BK * D; idx += PF_THREADS) {
            const int r = idx / D, c = idx - r * D;
            Ks[r * (D + 1) + c] = koff[r] >= 0 ? ldf(cache_k + koff[r] + c) : 0.f;
        }
        for (int idx = tid; idx < BK * Dv; idx += PF_THREADS) {
            const int r = idx / Dv, c = idx - r * Dv;
            Vs[idx] = voff[r] >= 0 ? ldf(cache_v + voff[r] + c) : 0.f;
        }
        __syncthreads();
        float s[4];
        float tmax = -INFINITY;
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const int kj = sub + 8 * m;
            const int j = k0 + kj;
            const float* qr = Qs + qi * D;
            const float* kr = Ks + kj * (D + 1);
            float d = 0.f;
            for (int c = 0; c < D; ++c) d = fmaf(qr[c], kr[c], d);
            const int dist = p_i - j;
            const bool vis = row_ok && dist >= 0 && (window <= 0 || dist < window || j < keep_first);
            s[m] = vis ? d - slope * (float)dist : -INFINITY;
            tmax = fmaxf(tmax, s[m]);
        }
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
        const float m_new = fmaxf(m_i, tmax);
        const float alpha = (m_new == -INFINITY) ? 1.f : expf(m_i - m_new);
        float tsum = 0.f;
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const float p = (s[m] == -INFINITY) ? 0.f : expf(s[m] - m_new);
            Ps[qi * BK + sub + 8 * m] = p;
            tsum += p;
        }
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) tsum += __shfl_xor_sync(0xffffffffu, tsum, o);
        l_i = l_i * alpha + tsum;
        m_i = m_new;
        __syncwarp();                        // the 8 threads of a query row are lanes of one warp
        const float* pr = Ps + qi * BK;
#pragma unroll
        for (int m = 0; m < MAXC; ++m) {
            if (m < nc) {
                const int c = sub + 8 * m;
                float a = acc[m] * alpha;
                if (c < Dv) {
                    for (int kj = 0; kj < BK; ++kj) a = fmaf(pr[kj], Vs[kj * Dv + c], a);
                }
                acc[m] = a;
            }
        }
    }
    if (q0 + qi < Tn) {
        const float inv = (row_ok && l_i > 0.f) ? 1.f / l_i : 0.f;
#pragma unroll
        for (int m = 0; m < MAXC; ++m) {
            if (m < nc) {
                const int c = sub + 8 * m;
                if (c < Dv) stf(orow + c, acc[m] * inv);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------------
constexpr int DEC_WARPS = 8, DEC_R = 8, DEC_MV = 8;   // query heads per CTA, value columns per lane (Dv <= 256)

template <typename T>
__global__ void __launch_bounds__(DEC_WARPS * 32)
window_attn_decode_kernel(const T* __restrict__ q, const T* __restrict__ cache_k, const T* __restrict__ cache_v,
                          CacheAddr ka, CacheAddr va, T* __restrict__ out, const int* __restrict__ positions,
                          const int* __restrict__ seq_ids, const float* __restrict__ slopes, int H, int G, int D, int Dv,
                          float scale, int window, int keep_first, int groups_per_kv) {
    extern __shared__ float smem[];
    const int R_all = H / G;
    const int g = blockIdx.x / groups_per_kv, sub_group = blockIdx.x % groups_per_kv;
    const int b = blockIdx.y;
    const int r0 = sub_group * DEC_R;
    const int R = min(DEC_R, R_all - r0);
    const int h0 = g * R_all + r0;
    float* Qs = smem;                                   // [DEC_R][D]
    float* Ms = Qs + DEC_R * D;                         // [DEC_WARPS][DEC_R][Dv + 2]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int p = positions[b];
    const int line = seq_ids != nullptr ? seq_ids[b] : b;
    for (int idx = tid; idx < R * D; idx += DEC_WARPS * 32) {
        const int r = idx / D, c = idx - r * D;
        Qs[idx] = ldf(q + ((long long)b * H + h0 + r) * D + c) * scale;
    }
    __syncthreads();
    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    const int n_sink = min(keep_first, lo);
    const int nk = n_sink + (p - lo + 1);
    float m_r[DEC_R], l_r[DEC_R], sl[DEC_R];
    float acc[DEC_R][DEC_MV];
#pragma unroll
    for (int r = 0; r < DEC_R; ++r) {
        m_r[r] = -INFINITY;
        l_r[r] = 0.f;
        sl[r] = (slopes != nullptr && r < R) ? slopes[h0 + r] : 0.f;
#pragma unroll
        for (int m = 0; m < DEC_MV; ++m) acc[r][m] = 0.f;
    }
    for (int i = warp; i < nk; i += DEC_WARPS) {
        const int j = i < n_sink ? i : lo + (i - n_sink);
        const T* kr = cache_k + ka.row(line, g, j);
        const T* vr = cache_v + va.row(line, g, j);
        float d[DEC_R];
#pragma unroll
        for (int r = 0; r < DEC_R; ++r) d[r] = 0.f;
        for (int c = lane; c < D; c += 32) {
            const float kv = ldf(kr + c);
#pragma unroll
            for (int r = 0; r < DEC_R; ++r)
                if (r < R) d[r] = fmaf(Qs[r * D + c], kv, d[r]);
        }
        float vv[DEC_MV];
#pragma unroll
        for (int m = 0; m < DEC_MV; ++m) {
            const int c = lane + 32 * m;
            vv[m] = c < Dv ? ldf(vr + c) : 0.f;
        }
        const float dist = (float)(p - j);
#pragma unroll
        for (int r = 0; r < DEC_R; ++r) {
            if (r < R) {
                const float s = warp_sum(d[r]) - sl[r] * dist;
                const float m_new = fmaxf(m_r[r], s);
                const float alpha = expf(m_r[r] - m_new);      // exp(-inf) = 0 on the first key
                const float pw = expf(s - m_new);
                l_r[r] = l_r[r] * alpha + pw;
                m_r[r] = m_new;
#pragma unroll
                for (int m = 0; m < DEC_MV; ++m) acc[r][m] = fmaf(pw, vv[m], acc[r][m] * alpha);
            }
        }
    }
    const int stride = Dv + 2;
#pragma unroll
    for (int r = 0; r < DEC_R; ++r) {
        if (r < R) {
            float* dst = Ms + ((long long)warp * DEC_R + r) * stride;
#pragma unroll
            for (int m = 0; m < DEC_MV; ++m) {
                const int c = lane + 32 * m;
                if (c < Dv) dst[c] = acc[r][m];
            }
            if (lane == 0) {
                dst[Dv] = m_r[r];
                dst[Dv + 1] = l_r[r];
            }
        }
    }
    __syncthreads();
    for (int idx = tid; idx < R * Dv; idx += DEC_WARPS * 32) {
        const int r = idx / Dv, c = idx - r * Dv;
        float mx = -INFINITY;
        for (int w = 0; w < DEC_WARPS; ++w) mx = fmaxf(mx, Ms[((long long)w * DEC_R + r) * stride + Dv]);
        float num = 0.f, den = 0.f;
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float* src = Ms + ((long long)w * DEC_R + r) * stride;
            const float mw = src[Dv];
            if (mw == -INFINITY) continue;
            const float f = expf(mw - mx);
            num = fmaf(f, src[c], num);
            den = fmaf(f, src[Dv + 1], den);
        }
        stf(out + ((long long)b * H + h0 + r) * Dv + c, den > 0.f ? num / den : 0.f);
    }
}

CacheAddr make_addr(long long stride_line, long long stride_head, const int* block_table, int page_size, int table_cols,
                    int row_dim) {
    CacheAddr a;
    a.stride_line = stride_line;
    a.stride_head = stride_head;
    a.block_table = block_table;
    a.page_size = page_size > 0 ? page_size : 1;
    a.table_cols = table_cols;
    a.row_dim = row_dim;
    return a;
}

template <typename T>
int launch_prefill(const void* q, const void* ck, const void* cv, CacheAddr ka, CacheAddr va, void* out,
                   const int* q_start, const int* n_new, const int* seq_ids, const float* slopes, int B, int Tn, int H,
                   int G, int D, int Dv, float scale, int window, int keep_first, cudaStream_t st) {
    const size_t smem = (size_t)(BQ * D + BK * (D + 1) + BK * Dv + BQ * BK) * sizeof(float);
    auto kern = window_attn_prefill_kernel<T>;
    if (smem > 48 * 1024) NXD_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((Tn + BQ - 1) / BQ, H, B);
    kern<<<grid, PF_THREADS, smem, st>>>((const T*)q, (const T*)ck, (const T*)cv, ka, va, (T*)out, q_start, n_new,
                                         seq_ids, slopes, Tn, H, G, D, Dv, scale, window, keep_first);
    NXD_LAUNCH_CHECK();
    return 0;
}

template <typename T>
int launch_decode(const void* q, const void* ck, const void* cv, CacheAddr ka, CacheAddr va, void* out,
                  const int* positions, const int* seq_ids, const float* slopes, int B, int H, int G, int D, int Dv,
                  float scale, int window, int keep_first, cudaStream_t st) {
    const int R_all = H / G;
    const int groups = (R_all + DEC_R - 1) / DEC_R;
    const size_t smem = (size_t)(DEC_R * D + DEC_WARPS * DEC_R * (Dv + 2)) * sizeof(float);
    auto kern = window_attn_decode_kernel<T>;
    if (smem > 48 * 1024) NXD_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid(G * groups, B);
    kern<<<grid, DEC_WARPS * 32, smem, st>>>((const T*)q, (const T*)ck, (const T*)cv, ka, va, (T*)out, positions, seq_ids,
                                             slopes, H, G, D, Dv, scale, window, keep_first, groups);
    NXD_LAUNCH_CHECK();
    return 0;
}

}  // namespace

// dtype: 0 = bf16, 1 = fp32 (projection output, q, cache and attention output share it).  qkv: [B * Tn, ld] rows laid
// out as H query heads of D, then (has_kv) G key heads of D and G value heads of Dv.  q_start [B]: position of the first
// new token of every row; n_new [B] or NULL: how many of the Tn rows are real (the others are padding and write
// nothing); seq_ids [B] or NULL: cache line of every row.  max_pos: rows of a cache line.
NXD_API int nxd_qk_norm_cache_write(int dtype, const void* qkv, long long ld, void* q_out, void* cache_k, void* cache_v,
                                    long long k_stride_line, long long k_stride_head, long long v_stride_line,
                                    long long v_stride_head, const int* block_table, int page_size, int table_cols,
                                    const int* q_start, const int* n_new, const int* seq_ids, int B, int Tn, int H, int G,
                                    int D, int Dv, int has_kv, int normalize, float eps, int max_pos, void* stream) {
    const long long units = (long long)B * Tn * (H + (has_kv ? 2 * G : 0));
    if (units == 0) return 0;
    const CacheAddr ka = make_addr(k_stride_line, k_stride_head, block_table, page_size, table_cols, D);
    const CacheAddr va = make_addr(v_stride_line, v_stride_head, block_table, page_size, table_cols, Dv);
    const int wpb = 8;
    const unsigned blocks = (unsigned)((units + wpb - 1) / wpb);
    if (dtype == 0)
        qk_norm_cache_write_kernel<bf16><<<blocks, wpb * 32, 0, (cudaStream_t)stream>>>(
            (const bf16*)qkv, ld, (bf16*)q_out, (bf16*)cache_k, (bf16*)cache_v, ka, va, q_start, n_new, seq_ids, units, Tn,
            H, G, D, Dv, has_kv, normalize, eps, max_pos);
    else
        qk_norm_cache_write_kernel<float><<<blocks, wpb * 32, 0, (cudaStream_t)stream>>>(
            (const float*)qkv, ld, (float*)q_out, (float*)cache_k, (float*)cache_v, ka, va, q_start, n_new, seq_ids, units,
            Tn, H, G, D, Dv, has_kv, normalize, eps, max_pos);
    NXD_LAUNCH_CHECK();
    return 0;
}

// q [B, Tn, H, D] -> out [B, Tn, H, Dv]; the keys and values of positions [0, q_start[b] + n_new[b]) are read from the
// cache (the new tokens' rows must have been written before).  slopes [H] fp32 or NULL; window <= 0: plain causal.
NXD_API int nxd_window_attn_prefill(int dtype, const void* q, const void* cache_k, const void* cache_v,
                                    long long k_stride_line, long long k_stride_head, long long v_stride_line,
                                    long long v_stride_head, const int* block_table, int page_size, int table_cols,
                                    void* out, const int* q_start, const int* n_new, const int* seq_ids,
                                    const float* slopes, int B, int Tn, int H, int G, int D, int Dv, float scale,
                                    int window, int keep_first, void* stream) {
    NXD_REQUIRE(G > 0 && H % G == 0, "window attention: %d query heads over %d key/value heads", H, G);
    NXD_REQUIRE(Dv <= MAXC * 8, "window attention: value size %d above %d", Dv, MAXC * 8);
    if (B * Tn == 0) return 0;
    const CacheAddr ka = make_addr(k_stride_line, k_stride_head, block_table, page_size, table_cols, D);
    const CacheAddr va = make_addr(v_stride_line, v_stride_head, block_table, page_size, table_cols, Dv);
    if (dtype == 0)
        return launch_prefill<bf16>(q, cache_k, cache_v, ka, va, out, q_start, n_new, seq_ids, slopes, B, Tn, H, G, D, Dv,
                                    scale, window, keep_first, (cudaStream_t)stream);
    return launch_prefill<float>(q, cache_k, cache_v, ka, va, out, q_start, n_new, seq_ids, slopes, B, Tn, H, G, D, Dv,
                                 scale, window, keep_first, (cudaStream_t)stream);
}

// q [B, H, D] of one new token per row at positions[b] (its key and value already in the cache) -> out [B, H, Dv].
NXD_API int nxd_window_attn_decode(int dtype, const void* q, const void* cache_k, const void* cache_v,
                                   long long k_stride_line, long long k_stride_head, long long v_stride_line,
                                   long long v_stride_head, const int* block_table, int page_size, int table_cols,
                                   void* out, const int* positions, const int* seq_ids, const float* slopes, int B, int H,
                                   int G, int D, int Dv, float scale, int window, int keep_first, void* stream) {
    NXD_REQUIRE(G > 0 && H % G == 0, "window attention: %d query heads over %d key/value heads", H, G);
    NXD_REQUIRE(Dv <= DEC_MV * 32, "window attention: value size %d above %d", Dv, DEC_MV * 32);
    if (B == 0) return 0;
    const CacheAddr ka = make_addr(k_stride_line, k_stride_head, block_table, page_size, table_cols, D);
    const CacheAddr va = make_addr(v_stride_line, v_stride_head, block_table, page_size, table_cols, Dv);
    if (dtype == 0)
        return launch_decode<bf16>(q, cache_k, cache_v, ka, va, out, positions, seq_ids, slopes, B, H, G, D, Dv, scale,
                                   window, keep_first, (cudaStream_t)stream);
    return launch_decode<float>(q, cache_k, cache_v, ka, va, out, positions, seq_ids, slopes, B, H, G, D, Dv, scale,
                                window, keep_first, (cudaStream_t)stream);
}
