// Latent (compressed key/value) attention: what a step does to the fused projection output before the attention
// kernel runs.
//
// The projection row of a token holds H query heads laid out [dim un-rotated | rot_dim rotated] at column q_off and, at
// column kv_off, kv_rank compressed key/value columns followed by rot_dim columns of ONE rotated key part shared by all
// heads.  Only the normalised compressed columns c and the rotated key part are cached: cache row = [c | k_rot].  Since
//   score_h(i, j) = <q_nope_h, W_uk_h c_j> + <q_rot_h, k_rot_j> = <[W_uk_h^T q_nope_h | q_rot_h], [c_j | k_rot_j]>
// every head attends to the same cache rows with an "absorbed" query, and the value is the c part of the row; the
// per-head value projection W_uv_h follows the attention.
//
//   latent_prep   one warp per (token, unit): units 0 .. H-1 copy the un-rotated query columns to q_nope and write the
//                 rotated query columns (pairs (2i, 2i+1) turned by the angle of (position, i)) to q_rot; unit H
//                 divides the compressed columns by their root mean square (fp32, eps inside the root), multiplies by
//                 the norm weight, rotates the shared key part and writes the cache row at (line, position).
//                 Padding tokens (t >= n_new[b]) write no cache row.
//   latent_decode one new token per row over wide latent rows (bf16, tensor cores): one CTA per (16 query heads, row,
//                 context split).  The 64-row tiles of the line stream through shared memory ONCE per CTA; each of the
//                 four warps scores 16 of the tile's rows (mma.sync m16n8k16, the query heads are the 16 MMA rows, the
//                 query fragments re-read from shared memory at every step of the 576 / 288 key columns), the tile's
//                 row maxima and the bf16 probabilities meet in shared memory, and each warp accumulates its own
//                 quarter of the value columns -- which are the first columns of the same tile rows, so nothing else is
//                 loaded.  With more than one context split the un-normalised partial results (fp32) are merged by
//                 latent_decode_merge, which also adds the sink logit to the denominator.
#include "common.cuh"
#include "mma_sync.cuh"

namespace {

__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const bf16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

template <typename T>
__global__ void latent_prep_kernel(const T* __restrict__ proj, long long ld, int q_off, int kv_off,
                                   T* __restrict__ q_nope, long long nope_head, T* __restrict__ q_rot, long long rot_head,
                                   T* __restrict__ cache, long long stride_line, long long row_pitch,
                                   const int* __restrict__ block_table, int page_size, int table_cols,
                                   const float* __restrict__ c_weight, const float* __restrict__ rope_cos,
                                   const float* __restrict__ rope_sin, const int* __restrict__ q_start,
                                   const int* __restrict__ n_new, const int* __restrict__ seq_ids, long long units,
                                   int Tn, int H, int dim, int rot, int rank, float eps, int max_pos) {
    const int lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= units) return;
    const long long n = unit / (H + 1);
    const int u = (int)(unit % (H + 1));
    const int b = (int)(n / Tn), t = (int)(n % Tn);
    const long long pos = (long long)q_start[b] + t;
    const float* cs = rope_cos + pos * (rot / 2);
    const float* sn = rope_sin + pos * (rot / 2);
    const T* row = proj + n * ld;
    if (u < H) {
        const T* src = row + q_off + (long long)u * (dim + rot);
        T* d0 = q_nope + (n * H + u) * nope_head;
        for (int i = lane; i < dim; i += 32) d0[i] = src[i];
        T* d1 = q_rot + (n * H + u) * rot_head;
        for (int i = lane; i < rot / 2; i += 32) {
            const float a = ldf(src + dim + 2 * i), c = ldf(src + dim + 2 * i + 1);
            stf(d1 + 2 * i, a * cs[i] - c * sn[i]);
            stf(d1 + 2 * i + 1, c * cs[i] + a * sn[i]);
        }
        return;
    }
    if ((n_new != nullptr && t >= n_new[b]) || pos >= max_pos) return;
    const int line = seq_ids != nullptr ? seq_ids[b] : b;
    T* dst;
    if (block_table != nullptr) {
        const int page = block_table[(long long)line * table_cols + pos / page_size];
        dst = cache + (long long)page * stride_line + (pos % page_size) * row_pitch;
    } else {
        dst = cache + (long long)line * stride_line + pos * row_pitch;
    }
    const T* src = row + kv_off;
    float ss = 0.f;
    for (int i = lane; i < rank; i += 32) {
        const float v = ldf(src + i);
        ss += v * v;
    }
    ss = warp_sum(ss);
    const float r = 1.f / sqrtf(ss / (float)rank + eps);
    for (int i = lane; i < rank; i += 32) stf(dst + i, ldf(src + i) * r * c_weight[i]);
    for (int i = lane; i < rot / 2; i += 32) {
        const float a = ldf(src + rank + 2 * i), c = ldf(src + rank + 2 * i + 1);
        stf(dst + rank + 2 * i, a * cs[i] - c * sn[i]);
        stf(dst + rank + 2 * i + 1, c * cs[i] + a * sn[i]);
    }
}

constexpr int LD_MK = 64, LD_THREADS = 128, LD_ROWS = 16;

template <int D, int DV>
__global__ void __launch_bounds__(LD_THREADS)
latent_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ cache, long long stride_line, long long row_pitch,
                     const int* __restrict__ block_table, int page_size, int table_cols, bf16* __restrict__ out,
                     float* __restrict__ partial, const int* __restrict__ positions, const int* __restrict__ seq_ids,
                     const float* __restrict__ sinks, int H, float scale, int nsplit) {
    constexpr int LDK = D + 8, CK = D / 8, LDP = LD_MK + 8, VW = DV / 4;     // VW: value columns per warp
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);       // [16][LDK]
    bf16* Ks = Qs + LD_ROWS * LDK;                      // [2][64][LDK]
    bf16* Ps = Ks + 2 * LD_MK * LDK;                    // [16][LDP]
    __shared__ long long koff[2][LD_MK];
    __shared__ float Mx[4][LD_ROWS];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int h0 = blockIdx.x * LD_ROWS, b = blockIdx.y, z = blockIdx.z;
    const int R = min(LD_ROWS, H - h0);
    const int p = positions[b];
    const int line = seq_ids != nullptr ? seq_ids[b] : b;
    const int tiles = p / LD_MK + 1;
    const int per = (tiles + nsplit - 1) / nsplit;
    const int t_lo = z * per, t_hi = min(tiles, t_lo + per);          // this CTA's tiles [t_lo, t_hi)
    const int n_tiles = max(0, t_hi - t_lo);
    const uint32_t qs_addr = (uint32_t)__cvta_generic_to_shared(Qs);
    const uint32_t ks_addr = (uint32_t)__cvta_generic_to_shared(Ks);
    const uint32_t ps_addr = (uint32_t)__cvta_generic_to_shared(Ps);

    constexpr float LOG2E = 1.4426950408889634f;
    const float sc2 = scale * LOG2E;
    const int r_lo = lane >> 2;
    const bool ok0 = r_lo < R, ok1 = r_lo + 8 < R;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float o[VW / 8][4];
#pragma unroll
    for (int i = 0; i < VW / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    if (n_tiles > 0) {
        for (int idx = tid; idx < LD_ROWS * CK; idx += LD_THREADS) {
            const int r = idx / CK, c = idx - r * CK;
            const bool ok = r < R;
            mma::cp_async16(qs_addr + (r * LDK + c * 8) * 2, ok ? q + ((long long)b * H + h0 + r) * D + c * 8 : q, ok);
        }
        auto issue = [&](int n, int buf) {
            const int kt = t_lo + n;
            if (tid < LD_MK) {
                const int pos = kt * LD_MK + tid;
                long long off = -1;
                if (pos <= p) {
                    if (block_table != nullptr)
                        off = (long long)block_table[(long long)line * table_cols + pos / page_size] * stride_line +
                              (long long)(pos % page_size) * row_pitch;
                    else
                        off = (long long)line * stride_line + (long long)pos * row_pitch;
                }
                koff[buf][tid] = off;
            }
            __syncthreads();
            for (int idx = tid; idx < LD_MK * CK; idx += LD_THREADS) {
                const int r = idx / CK, c = idx - r * CK;
                const bool ok = koff[buf][r] >= 0;
                mma::cp_async16(ks_addr + ((buf * LD_MK + r) * LDK + c * 8) * 2, ok ? cache + koff[buf][r] + c * 8 : cache, ok);
            }
            mma::cp_async_commit();
        };
        issue(0, 0);
        for (int n = 0; n < n_tiles; ++n) {
            const int buf = n & 1;
            if (n + 1 < n_tiles) {
                issue(n + 1, buf ^ 1);
                mma::cp_async_wait<1>();
            } else {
                mma::cp_async_wait<0>();
            }
            __syncthreads();
            const int k0 = (t_lo + n) * LD_MK + warp * 16;               // this warp's 16 rows of the tile
            float s[2][4];
            s[0][0] = s[0][1] = s[0][2] = s[0][3] = s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.f;
            const uint32_t kb_addr = ks_addr + buf * LD_MK * LDK * 2;
#pragma unroll 4
            for (int kk = 0; kk < D / 16; ++kk) {
                uint32_t bfr[4], qa[4];
                const int row = warp * 16 + (lane & 7) + (lane >> 4) * 8;
                mma::ldsm_x4(bfr, kb_addr + (row * LDK + kk * 16 + ((lane >> 3) & 1) * 8) * 2);
                mma::ldsm_x4(qa, qs_addr + ((lane & 15) * LDK + kk * 16 + (lane >> 4) * 8) * 2);
                mma::mma16816(s[0], qa, bfr[0], bfr[1]);
                mma::mma16816(s[1], qa, bfr[2], bfr[3]);
            }
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = k0 + i * 8 + (lane & 3) * 2 + (e & 1);
                    const bool vis = ((e & 2) ? ok1 : ok0) && j <= p;
                    const float v = vis ? s[i][e] * sc2 : -INFINITY;
                    s[i][e] = v;
                    if (e & 2) mx1 = fmaxf(mx1, v); else mx0 = fmaxf(mx0, v);
                }
            }
            mx0 = mma::quad_max(mx0);
            mx1 = mma::quad_max(mx1);
            if ((lane & 3) == 0) {
                Mx[warp][r_lo] = mx0;
                Mx[warp][r_lo + 8] = mx1;
            }
            __syncthreads();
            const float t0 = fmaxf(fmaxf(Mx[0][r_lo], Mx[1][r_lo]), fmaxf(Mx[2][r_lo], Mx[3][r_lo]));
            const float t1 = fmaxf(fmaxf(Mx[0][r_lo + 8], Mx[1][r_lo + 8]), fmaxf(Mx[2][r_lo + 8], Mx[3][r_lo + 8]));
            const float mn0 = fmaxf(m0, t0), mn1 = fmaxf(m1, t1);
            const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
            const float a0 = exp2f(m0 - ms0), a1 = exp2f(m1 - ms1);
            m0 = mn0;
            m1 = mn1;
            float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const float p00 = exp2f(s[i][0] - ms0), p01 = exp2f(s[i][1] - ms0);
                const float p10 = exp2f(s[i][2] - ms1), p11 = exp2f(s[i][3] - ms1);
                ps0 += p00 + p01;
                ps1 += p10 + p11;
                const int c = warp * 16 + i * 8 + (lane & 3) * 2;
                *reinterpret_cast<uint32_t*>(Ps + r_lo * LDP + c) = mma::pack2(p00, p01);
                *reinterpret_cast<uint32_t*>(Ps + (r_lo + 8) * LDP + c) = mma::pack2(p10, p11);
            }
            l0 = l0 * a0 + ps0;
            l1 = l1 * a1 + ps1;
#pragma unroll
            for (int i = 0; i < VW / 8; ++i) {
                o[i][0] *= a0;
                o[i][1] *= a0;
                o[i][2] *= a1;
                o[i][3] *= a1;
            }
            __syncthreads();                                  // all probabilities of the tile are in Ps
#pragma unroll
            for (int kb = 0; kb < LD_MK / 16; ++kb) {
                uint32_t pa[4];
                mma::ldsm_x4(pa, ps_addr + ((lane & 15) * LDP + kb * 16 + (lane >> 4) * 8) * 2);
#pragma unroll
                for (int dj = 0; dj < VW / 16; ++dj) {
                    uint32_t bfr[4];
                    const int row = kb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                    mma::ldsm_x4_t(bfr, kb_addr + (row * LDK + warp * VW + dj * 16 + (lane >> 4) * 8) * 2);
                    mma::mma16816(o[2 * dj], pa, bfr[0], bfr[1]);
                    mma::mma16816(o[2 * dj + 1], pa, bfr[2], bfr[3]);
                }
            }
            __syncthreads();                                  // tile buffer, Ps and Mx are free again
        }
    }
    // row sums: every warp summed the probabilities of its own 16 rows of each tile
    l0 = mma::quad_sum(l0);
    l1 = mma::quad_sum(l1);
    if ((lane & 3) == 0) {
        Mx[warp][r_lo] = l0;
        Mx[warp][r_lo + 8] = l1;
    }
    __syncthreads();
    l0 = Mx[0][r_lo] + Mx[1][r_lo] + Mx[2][r_lo] + Mx[3][r_lo];
    l1 = Mx[0][r_lo + 8] + Mx[1][r_lo + 8] + Mx[2][r_lo + 8] + Mx[3][r_lo + 8];
    if (nsplit == 1) {
        if (sinks != nullptr) {
            if (ok0) l0 += exp2f(sinks[h0 + r_lo] * LOG2E - (m0 == -INFINITY ? 0.f : m0));
            if (ok1) l1 += exp2f(sinks[h0 + r_lo + 8] * LOG2E - (m1 == -INFINITY ? 0.f : m1));
        }
        const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
#pragma unroll
        for (int i = 0; i < VW / 8; ++i) {
            const int c = warp * VW + i * 8 + (lane & 3) * 2;
            if (ok0) *reinterpret_cast<uint32_t*>(out + ((long long)b * H + h0 + r_lo) * DV + c) = mma::pack2(o[i][0] * i0, o[i][1] * i0);
            if (ok1)
                *reinterpret_cast<uint32_t*>(out + ((long long)b * H + h0 + r_lo + 8) * DV + c) = mma::pack2(o[i][2] * i1, o[i][3] * i1);
        }
        return;
    }
    // partial[b, h, z, :] = [o (DV, un-normalised) | m | l]
    float* w0 = partial + (((long long)b * H + h0 + r_lo) * nsplit + z) * (DV + 2);
    float* w1 = partial + (((long long)b * H + h0 + r_lo + 8) * nsplit + z) * (DV + 2);
#pragma unroll
    for (int i = 0; i < VW / 8; ++i) {
        const int c = warp * VW + i * 8 + (lane & 3) * 2;
        if (ok0) {
            w0[c] = o[i][0];
            w0[c + 1] = o[i][1];
        }
        if (ok1) {
            w1[c] = o[i][2];
            w1[c + 1] = o[i][3];
        }
    }
    if (warp == 0 && (lane & 3) == 0) {
        if (ok0) {
            w0[DV] = m0;
            w0[DV + 1] = l0;
        }
        if (ok1) {
            w1[DV] = m1;
            w1[DV + 1] = l1;
        }
    }
}

// out[b, h, :] = sum_z 2^(m_z - M) o_z / (sum_z 2^(m_z - M) l_z + 2^(sink_h log2e - M)),  M = max_z m_z
__global__ void latent_decode_merge_kernel(const float* __restrict__ partial, const float* __restrict__ sinks,
                                           bf16* __restrict__ out, int H, int DV, int nsplit) {
    const int h = blockIdx.x, b = blockIdx.y;
    const float* src = partial + ((long long)b * H + h) * nsplit * (DV + 2);
    constexpr float LOG2E = 1.4426950408889634f;
    float mx = -INFINITY;
    for (int zz = 0; zz < nsplit; ++zz) mx = fmaxf(mx, src[zz * (DV + 2) + DV]);
    const float ms = mx == -INFINITY ? 0.f : mx;
    float den = sinks != nullptr ? exp2f(sinks[h] * LOG2E - ms) : 0.f;
    for (int zz = 0; zz < nsplit; ++zz) {
        const float mz = src[zz * (DV + 2) + DV];
        if (mz != -INFINITY) den = fmaf(exp2f(mz - ms), src[zz * (DV + 2) + DV + 1], den);
    }
    const float inv = den > 0.f ? 1.f / den : 0.f;
    for (int c = threadIdx.x; c < DV; c += blockDim.x) {
        float num = 0.f;
        for (int zz = 0; zz < nsplit; ++zz) {
            const float mz = src[zz * (DV + 2) + DV];
            if (mz != -INFINITY) num = fmaf(exp2f(mz - ms), src[zz * (DV + 2) + c], num);
        }
        out[((long long)b * H + h) * DV + c] = __float2bfloat16_rn(num * inv);
    }
}

template <int D, int DV>
int launch_latent_decode(const void* q, const void* cache, long long stride_line, long long row_pitch,
                         const int* block_table, int page_size, int table_cols, void* out, float* partial,
                         const int* positions, const int* seq_ids, const float* sinks, int B, int H, float scale, int nsplit,
                         cudaStream_t st) {
    const size_t smem = (size_t)(LD_ROWS * (D + 8) + 2 * LD_MK * (D + 8) + LD_ROWS * (LD_MK + 8)) * sizeof(bf16);
    auto kern = latent_decode_kernel<D, DV>;
    NXD_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((H + LD_ROWS - 1) / LD_ROWS, B, nsplit);
    kern<<<grid, LD_THREADS, smem, st>>>((const bf16*)q, (const bf16*)cache, stride_line, row_pitch, block_table,
                                         page_size > 0 ? page_size : 1, table_cols, (bf16*)out, partial, positions, seq_ids,
                                         sinks, H, scale, nsplit);
    NXD_LAUNCH_CHECK();
    if (nsplit > 1) {
        latent_decode_merge_kernel<<<dim3(H, B), 128, 0, st>>>(partial, sinks, (bf16*)out, H, DV, nsplit);
        NXD_LAUNCH_CHECK();
    }
    return 0;
}

}  // namespace

// bf16 token generation over latent rows: q [B, H, D] absorbed queries, cache rows of D columns (row_pitch elements
// apart) whose first Dv columns are the values; out [B, H, Dv] bf16; partial: fp32 scratch [B, H, nsplit, Dv + 2] (unused
// with nsplit == 1).  Returns 2 when no kernel is compiled for (D, Dv): the caller takes the general decode kernels.
NXD_API int nxd_latent_decode(const void* q, const void* cache, long long stride_line, long long row_pitch,
                              const int* block_table, int page_size, int table_cols, void* out, float* partial,
                              const int* positions, const int* seq_ids, const float* sinks, int B, int H, int D, int Dv,
                              float scale, int nsplit, void* stream) {
    if (B == 0) return 0;
    if ((stride_line % 8) || (row_pitch % 8) || ((uintptr_t)cache % 16) || ((uintptr_t)q % 16)) return 2;
    cudaStream_t st = (cudaStream_t)stream;
#define NXD_LD_CASE(DD, DDV)                                                                                            \
    if (D == DD && Dv == DDV)                                                                                           \
        return launch_latent_decode<DD, DDV>(q, cache, stride_line, row_pitch, block_table, page_size, table_cols, out, \
                                             partial, positions, seq_ids, sinks, B, H, scale, nsplit, st)
    NXD_LD_CASE(576, 512);
    NXD_LD_CASE(288, 256);
    NXD_LD_CASE(160, 128);
    NXD_LD_CASE(320, 256);
#undef NXD_LD_CASE
    return 2;
}

// dtype: 0 = bf16, 1 = fp32 (projection, queries and cache share it).  proj [B * Tn, ld].  q_nope: H heads per token,
// nope_head elements apart (>= dim); q_rot likewise (rot_head >= rot_dim): both may point into one wider buffer.
// cache [lines or pages, 1, rows, row_pitch] with row_pitch >= rank + rot_dim; block_table [lines, table_cols] or NULL.
// rope_cos / rope_sin [positions, rot_dim / 2] fp32.
NXD_API int nxd_latent_prep(int dtype, const void* proj, long long ld, int q_off, int kv_off, void* q_nope,
                            long long nope_head, void* q_rot, long long rot_head, void* cache, long long stride_line,
                            long long row_pitch, const int* block_table, int page_size, int table_cols,
                            const float* c_weight, const float* rope_cos, const float* rope_sin, const int* q_start,
                            const int* n_new, const int* seq_ids, int B, int Tn, int H, int dim, int rot, int rank,
                            float eps, int max_pos, void* stream) {
    const long long units = (long long)B * Tn * (H + 1);
    if (units == 0) return 0;
    NXD_REQUIRE(rot % 2 == 0, "latent attention: %d rotated dimensions", rot);
    const int wpb = 8;
    const unsigned blocks = (unsigned)((units + wpb - 1) / wpb);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == 0)
        latent_prep_kernel<bf16><<<blocks, wpb * 32, 0, st>>>(
            (const bf16*)proj, ld, q_off, kv_off, (bf16*)q_nope, nope_head, (bf16*)q_rot, rot_head, (bf16*)cache,
            stride_line, row_pitch, block_table, page_size > 0 ? page_size : 1, table_cols, c_weight, rope_cos, rope_sin,
            q_start, n_new, seq_ids, units, Tn, H, dim, rot, rank, eps, max_pos);
    else
        latent_prep_kernel<float><<<blocks, wpb * 32, 0, st>>>(
            (const float*)proj, ld, q_off, kv_off, (float*)q_nope, nope_head, (float*)q_rot, rot_head, (float*)cache,
            stride_line, row_pitch, block_table, page_size > 0 ? page_size : 1, table_cols, c_weight, rope_cos, rope_sin,
            q_start, n_new, seq_ids, units, Tn, H, dim, rot, rank, eps, max_pos);
    NXD_LAUNCH_CHECK();
    return 0;
}
