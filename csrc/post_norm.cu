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
