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
#include "common.cuh"

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

}  // namespace

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
