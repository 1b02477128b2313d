// RMS norm with a zero-centred weight, applied to a sublayer's OUTPUT and added to an fp32 residual stream:
//
//   n = y / sqrt(mean(y^2) + eps) * (1 + w);   x <- x + n  (x fp32, in place);   h = cast(x)   (optional)
//
// With x == NULL the kernel is the plain norm (h = cast(n)): the model's final norm.  One CTA per row, the row is read
// once into registers (up to 16 values per thread, above that it is re-read), statistics in fp32.
#include "common.cuh"

namespace {

__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const bf16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

constexpr int PN_THREADS = 128, PN_REG = 16;

template <typename TY, typename TW, typename TH>
__global__ void __launch_bounds__(PN_THREADS)
post_norm_kernel(const TY* __restrict__ y, const TW* __restrict__ w, float* __restrict__ x, TH* __restrict__ h, int W,
                 float eps, float offset) {
    __shared__ float red[32];
    const long long row = blockIdx.x;
    const TY* yr = y + row * W;
    float v[PN_REG];
    float ss = 0.f;
    const bool in_regs = W <= PN_REG * PN_THREADS;
    if (in_regs) {
#pragma unroll
        for (int i = 0; i < PN_REG; ++i) {
            const int c = threadIdx.x + i * PN_THREADS;
            v[i] = c < W ? ldf(yr + c) : 0.f;
            ss += v[i] * v[i];
        }
    } else {
        for (int c = threadIdx.x; c < W; c += PN_THREADS) {
            const float t = ldf(yr + c);
            ss += t * t;
        }
    }
    ss = block_sum(ss, red);
    const float r = 1.f / sqrtf(ss / (float)W + eps);
    if (in_regs) {
#pragma unroll
        for (int i = 0; i < PN_REG; ++i) {
            const int c = threadIdx.x + i * PN_THREADS;
            if (c < W) {
                float n = v[i] * r * (offset + ldf(w + c));
                if (x != nullptr) {
                    n += x[row * W + c];
                    x[row * W + c] = n;
                }
                if (h != nullptr) stf(h + row * W + c, n);
            }
        }
    } else {
        for (int c = threadIdx.x; c < W; c += PN_THREADS) {
            float n = ldf(yr + c) * r * (offset + ldf(w + c));
            if (x != nullptr) {
                n += x[row * W + c];
                x[row * W + c] = n;
            }
            if (h != nullptr) stf(h + row * W + c, n);
        }
    }
}

template <typename TY, typename TW, typename TH>
int launch(const void* y, const void* w, float* x, void* h, long long rows, int W, float eps, float offset,
           cudaStream_t st) {
    post_norm_kernel<TY, TW, TH><<<(unsigned)rows, PN_THREADS, 0, st>>>((const TY*)y, (const TW*)w, x, (TH*)h, W, eps,
                                                                        offset);
    NXD_LAUNCH_CHECK();
    return 0;
}


// Pre- and post-norm of one sublayer boundary in a single pass over an fp32 residual stream:
//
//   (y given)       x <- x + norm(y) * w_post                  (norm on the sublayer's output, x in place)
//   (w_next given)  h  = cast(norm(x) * w_next)                (the next sublayer's input)
//
// norm(v) = (v - mean(v)) / sqrt(var(v) + eps) with center != 0 (layer norm, weight only), v / sqrt(mean(v^2) + eps)
// otherwise.  One CTA per row; the row sits in shared memory, mean and variance are two separate fp32 reductions.
template <typename TY, typename TH>
__global__ void __launch_bounds__(PN_THREADS)
norm_chain_kernel(const TY* __restrict__ y, const float* __restrict__ w_post, float* __restrict__ x,
                  const float* __restrict__ w_next, TH* __restrict__ h, int W, float eps, int center) {
    extern __shared__ float rowbuf[];
    __shared__ float red[32];
    const long long row = blockIdx.x;
    float* xr = x + row * W;
    if (y != nullptr) {
        const TY* yr = y + row * W;
        float s = 0.f;
        for (int c = threadIdx.x; c < W; c += PN_THREADS) {
            const float v = ldf(yr + c);
            rowbuf[c] = v;
            s += v;
        }
        const float mean = center ? block_sum(s, red) / (float)W : 0.f;
        float ss = 0.f;
        for (int c = threadIdx.x; c < W; c += PN_THREADS) {
            const float d = rowbuf[c] - mean;
            ss += d * d;
        }
        const float r = 1.f / sqrtf(block_sum(ss, red) / (float)W + eps);
        for (int c = threadIdx.x; c < W; c += PN_THREADS) {
            const float v = xr[c] + (rowbuf[c] - mean) * r * w_post[c];
            xr[c] = v;
            rowbuf[c] = v;
        }
    } else {
        for (int c = threadIdx.x; c < W; c += PN_THREADS) rowbuf[c] = xr[c];
    }
    if (w_next == nullptr || h == nullptr) return;
    float s = 0.f;
    for (int c = threadIdx.x; c < W; c += PN_THREADS) s += rowbuf[c];
    const float mean = center ? block_sum(s, red) / (float)W : 0.f;
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += PN_THREADS) {
        const float d = rowbuf[c] - mean;
        ss += d * d;
    }
    const float r = 1.f / sqrtf(block_sum(ss, red) / (float)W + eps);
    TH* hr = h + row * W;
    for (int c = threadIdx.x; c < W; c += PN_THREADS) stf(hr + c, (rowbuf[c] - mean) * r * w_next[c]);
}

template <typename TY, typename TH>
int launch_chain(const void* y, const float* w_post, float* x, const float* w_next, void* h, long long rows, int W,
                 float eps, int center, cudaStream_t st) {
    const size_t smem = (size_t)W * sizeof(float);
    auto kern = norm_chain_kernel<TY, TH>;
    if (smem > 48 * 1024) NXD_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<(unsigned)rows, PN_THREADS, smem, st>>>((const TY*)y, w_post, x, w_next, (TH*)h, W, eps, center);
    NXD_LAUNCH_CHECK();
    return 0;
}

}  // namespace

// y [rows, W] (y_dtype), w [W] (w_dtype), x [rows, W] fp32 or NULL, h [rows, W] (h_dtype) or NULL; dtypes: 0 bf16,
// 1 fp32.  offset is added to the weight (1 for a weight stored around zero, 0 for a plain weight).
NXD_API int nxd_post_norm_residual(int y_dtype, int w_dtype, int h_dtype, const void* y, const void* w, float* x, void* h,
                                   long long rows, int W, float eps, float offset, void* stream) {
    if (rows == 0) return 0;
    NXD_REQUIRE(rows < (1ll << 31), "post norm: %lld rows", rows);
    cudaStream_t st = (cudaStream_t)stream;
    const int key = (y_dtype << 2) | (w_dtype << 1) | h_dtype;
    switch (key) {
        case 0: return launch<bf16, bf16, bf16>(y, w, x, h, rows, W, eps, offset, st);
        case 1: return launch<bf16, bf16, float>(y, w, x, h, rows, W, eps, offset, st);
        case 2: return launch<bf16, float, bf16>(y, w, x, h, rows, W, eps, offset, st);
        case 3: return launch<bf16, float, float>(y, w, x, h, rows, W, eps, offset, st);
        case 4: return launch<float, bf16, bf16>(y, w, x, h, rows, W, eps, offset, st);
        case 5: return launch<float, bf16, float>(y, w, x, h, rows, W, eps, offset, st);
        case 6: return launch<float, float, bf16>(y, w, x, h, rows, W, eps, offset, st);
        default: return launch<float, float, float>(y, w, x, h, rows, W, eps, offset, st);
    }
}

// x [rows, W] fp32 stream (updated in place when y is given); y [rows, W] (y_dtype) or NULL; w_post, w_next [W] fp32 (or
// NULL); h [rows, W] (h_dtype) or NULL.  center: 1 = layer norm (mean removed), 0 = RMS norm.
NXD_API int nxd_norm_chain(int y_dtype, int h_dtype, const void* y, const float* w_post, float* x, const float* w_next,
                           void* h, long long rows, int W, float eps, int center, void* stream) {
    if (rows == 0) return 0;
    NXD_REQUIRE(rows < (1ll << 31), "norm chain: %lld rows", rows);
    NXD_REQUIRE((size_t)W * sizeof(float) <= 200 * 1024, "norm chain: width %d", W);
    cudaStream_t st = (cudaStream_t)stream;
    switch ((y_dtype << 1) | h_dtype) {
        case 0: return launch_chain<bf16, bf16>(y, w_post, x, w_next, h, rows, W, eps, center, st);
        case 1: return launch_chain<bf16, float>(y, w_post, x, w_next, h, rows, W, eps, center, st);
        case 2: return launch_chain<float, bf16>(y, w_post, x, w_next, h, rows, W, eps, center, st);
        default: return launch_chain<float, float>(y, w_post, x, w_next, h, rows, W, eps, center, st);
    }
}
