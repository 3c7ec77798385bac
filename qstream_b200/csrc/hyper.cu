// A residual stream kept as several copies ("hyper-connections"), and what touches it.
//
// The stream of a token is S vectors x_1 .. x_S of width D, stored side by side in one 32-bit row [S * D].  A
// sublayer reads one vector u = sum_s in[s] x_s, normed; its result y comes back into every copy at once:
//     x_t <- sum_s mix[s][t] x_s + out[t] * (scale . y),        scale: a vector of width D (layer scale), or none
// where y may itself be the sum of two branches with a constant factor each.  One kernel does a write (of the
// sublayer that has just finished), a read (for the sublayer that follows) with its RMS norm, or both in one pass
// over the row; the final read, with in = 1, gives the sum of the copies.  S = 1 with in = mix = out = 1 is the
// plain residual stream.  Everything is 32-bit; the normed vector is rounded once to the type asked for.
#include "common.cuh"

namespace {

constexpr int MAX_STREAMS = 8;

template <typename TY, typename TH>
__global__ void hyper_mix_norm_kernel(float* __restrict__ x, size_t ldx, int S, int D,
                                      const TY* __restrict__ y1, size_t ldy1, float c1,
                                      const TY* __restrict__ y2, size_t ldy2, float c2,
                                      const void* __restrict__ scale, int scale_dtype,
                                      const float* __restrict__ mix, const float* __restrict__ outw,
                                      const float* __restrict__ inw, const void* __restrict__ w, int w_dtype, float offset,
                                      float eps, TH* __restrict__ h, size_t ldh, int plain_sum) {
    extern __shared__ float u_of[];                     // [D] the vector that is read
    __shared__ float scratch[33];
    __shared__ float s_mix[MAX_STREAMS * MAX_STREAMS], s_out[MAX_STREAMS], s_in[MAX_STREAMS];
    grid_dep_launch();
    const bool write = y1 != nullptr;
    const bool read = h != nullptr;
    // the layers' constants are old: they are fetched before the wait for the previous kernel
    if (threadIdx.x < S * S) s_mix[threadIdx.x] = mix ? mix[threadIdx.x] : (threadIdx.x / S == threadIdx.x % S ? 1.f : 0.f);
    if (threadIdx.x < S) {
        s_out[threadIdx.x] = outw ? outw[threadIdx.x] : 1.f;
        s_in[threadIdx.x] = inw ? inw[threadIdx.x] : 1.f;
    }
    grid_dep_wait();
    __syncthreads();
    float* row = x + (size_t)blockIdx.x * ldx;
    float sq = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        float xs[MAX_STREAMS];
#pragma unroll
        for (int s = 0; s < MAX_STREAMS; ++s) xs[s] = s < S ? row[(size_t)s * D + i] : 0.f;
        if (write) {
            float y = c1 * to_f32(y1[(size_t)blockIdx.x * ldy1 + i]);
            if (y2) y = fmaf(c2, to_f32(y2[(size_t)blockIdx.x * ldy2 + i]), y);
            if (scale) y *= load_as_f32(scale, scale_dtype, i);
            float nx[MAX_STREAMS];
#pragma unroll
            for (int t = 0; t < MAX_STREAMS; ++t) {
                if (t < S) {
                    float a = 0.f;
                    for (int s = 0; s < S; ++s) a = fmaf(s_mix[s * S + t], xs[s], a);
                    nx[t] = fmaf(s_out[t], y, a);
                }
            }
#pragma unroll
            for (int t = 0; t < MAX_STREAMS; ++t)
                if (t < S) { xs[t] = nx[t]; row[(size_t)t * D + i] = nx[t]; }
        }
        if (read) {
            float u = 0.f;
            for (int s = 0; s < S; ++s) u = fmaf(s_in[s], xs[s], u);
            u_of[i] = u;
            sq = fmaf(u, u, sq);
        }
    }
    if (!read) return;
    if (plain_sum) {                                    // the vector as it is, no norm
        for (int i = threadIdx.x; i < D; i += blockDim.x) h[(size_t)blockIdx.x * ldh + i] = from_f32<TH>(u_of[i]);
        return;
    }
    const float total = block_sum(sq, scratch);
    const float rstd = 1.0f / sqrtf(total / (float)D + eps);
    for (int i = threadIdx.x; i < D; i += blockDim.x)
        h[(size_t)blockIdx.x * ldh + i] = from_f32<TH>(u_of[i] * rstd * (offset + load_as_f32(w, w_dtype, i)));
}

template <typename TY, typename TH>
int launch_hyper(float* x, long long ldx, int rows, int S, int D, const void* y1, long long ldy1, float c1, const void* y2,
                 long long ldy2, float c2, const void* scale, int scale_dtype, const float* mix, const float* outw,
                 const float* inw, const void* w, int w_dtype, float offset, float eps, void* h, long long ldh, int plain_sum,
                 cudaStream_t stream) {
    const int threads = D >= 2048 ? 256 : 128;
    const size_t smem = (size_t)D * sizeof(float);
    cudaError_t e = smem > 48 * 1024 ? cudaFuncSetAttribute(hyper_mix_norm_kernel<TY, TH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                                     : cudaSuccess;
    if (e == cudaSuccess)
        e = qs_launch_dependent(hyper_mix_norm_kernel<TY, TH>, dim3(rows), dim3(threads), smem, stream, x, (size_t)ldx, S, D,
                                (const TY*)y1, (size_t)ldy1, c1, (const TY*)y2, (size_t)ldy2, c2, scale, scale_dtype, mix, outw,
                                inw, w, w_dtype, offset, eps, (TH*)h, (size_t)ldh, plain_sum);
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "hyper_mix_norm: %s", cudaGetErrorString(e));
    return qs_check_launch("hyper_mix_norm");
}

// Every copy of the stream starts as the same vector: x [rows, S * D] <- S times src [rows, D].
__global__ void hyper_spread_kernel(float* __restrict__ x, size_t ldx, int S, int D, const float* __restrict__ src, size_t lds) {
    grid_dep_launch();
    grid_dep_wait();
    float* row = x + (size_t)blockIdx.x * ldx;
    const float* from = src + (size_t)blockIdx.x * lds;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const float v = from[i];
        for (int s = 0; s < S; ++s) row[(size_t)s * D + i] = v;
    }
}

}  // namespace

QS_API int qs_hyper_spread(float* x, long long ldx, int rows, int S, int D, const float* src, long long lds, cudaStream_t stream) {
    if (rows == 0) return QS_OK;
    QS_REQUIRE(rows > 0 && D > 0 && S >= 1, "hyper_spread: bad sizes");
    cudaError_t e = qs_launch_dependent(hyper_spread_kernel, dim3(rows), dim3(D >= 2048 ? 256 : 128), 0, stream, x, (size_t)ldx, S, D,
                                        src, (size_t)lds);
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "hyper_spread: %s", cudaGetErrorString(e));
    return qs_check_launch("hyper_spread");
}

// x [rows, S * D] float32, changed in place by the write (y1 given).  h [rows, D] given: the read, normed with w
// (offset + w) unless `plain_sum`.  mix [S * S] ([from][to]), outw [S], inw [S]: float32, each may be null (identity,
// ones, ones).  y1, y2 share a type (y_dtype); y2 and scale may be null.
QS_API int qs_hyper_mix_norm(float* x, long long ldx, int rows, int S, int D, const void* y1, long long ldy1, float c1,
                             const void* y2, long long ldy2, float c2, int y_dtype, const void* scale, int scale_dtype,
                             const float* mix, const float* outw, const float* inw, const void* w, int w_dtype,
                             float offset, float eps, void* h, int h_dtype, long long ldh, int plain_sum, cudaStream_t stream) {
    if (rows == 0) return QS_OK;
    QS_REQUIRE(rows > 0 && D > 0 && S >= 1 && S <= MAX_STREAMS, "hyper_mix_norm: %d copies of width %d (at most %d copies)", S, D, MAX_STREAMS);
    QS_REQUIRE(y1 || h, "hyper_mix_norm: neither a write nor a read");
    QS_REQUIRE(!h || plain_sum || w, "hyper_mix_norm: a normed read without a weight");
    QS_REQUIRE((size_t)D * sizeof(float) <= 200 * 1024, "hyper_mix_norm: width %d above the shared memory of a block", D);
    typedef __nv_bfloat16 bf16;
    if (!y1) y_dtype = QS_F32;
    if (!h) h_dtype = QS_F32;
#define GO(TY, TH) return launch_hyper<TY, TH>(x, ldx, rows, S, D, y1, ldy1, c1, y2, ldy2, c2, scale, scale_dtype, mix, outw, inw, \
                                               w, w_dtype, offset, eps, h, ldh, plain_sum, stream)
    if (y_dtype == QS_F32 && h_dtype == QS_F32) GO(float, float);
    if (y_dtype == QS_F32 && h_dtype == QS_BF16) GO(float, bf16);
    if (y_dtype == QS_BF16 && h_dtype == QS_BF16) GO(bf16, bf16);
    if (y_dtype == QS_BF16 && h_dtype == QS_F32) GO(bf16, float);
#undef GO
    return qs_fail(QS_ERR_INVALID_INPUT, "hyper_mix_norm: unknown types y=%d h=%d", y_dtype, h_dtype);
}
