// Attention through a latent: what a layer keeps per token is one normed latent vector c [kv_rank] and one rotated
// key part [rot_dim] that all heads share; keys and values of a head are linear maps of c.
//
// With the key map folded into the query (q' = W_uk^T q_unrotated) a head's score is q' . c + q_rot . k_rot, and
// its output is W_uv (sum_j p_j c_j): attention with ONE key head of size kv_rank + rot_dim whose values are the
// first kv_rank elements of the keys.  The kernels here prepare that form and leave the attention to the
// library's attention kernels:
//
//   latent_prepare   RMS norm of the query latent; RMS norm of the key latent and rotation of the shared key
//                    part, both written into the paged cache (keys [c | k_rot], values c)
//   latent_q_rotate  the rotated part of every head's query, moved behind the head's folded part
//   head_linear      one small matrix per head (the folded key map, the value map) for steps of few tokens
//
// The rotation pairs element i with i + dims/2 ("rotate half"): (u, v) -> (u cos a - v sin a, v cos a + u sin a)
// times `mag`, a = position * freq[i], with the frequencies given by the caller (any scaling of them is the
// caller's business); with `interleaved` the pairs are elements 2i and 2i + 1 instead.  Angles are taken in double
// precision, everything else in 32-bit, rounded once.
#include "common.cuh"

namespace {

template <typename T>
__global__ void latent_prepare_kernel(T* __restrict__ cq_out, size_t ldcq, const T* __restrict__ dq, size_t lddq,
                                      const void* __restrict__ wq, int wq_dtype, int q_rank,
                                      const T* __restrict__ dkv, size_t lddkv, const void* __restrict__ wkv, int wkv_dtype,
                                      int kv_rank, int rot_dim, int rot_dims, const double* __restrict__ freq, float mag,
                                      float eps, const int32_t* __restrict__ tok_slot, const int32_t* __restrict__ tok_pos,
                                      const int32_t* __restrict__ page_table, int max_pages, int page_shift,
                                      T* __restrict__ k_cache, T* __restrict__ v_cache, int32_t* __restrict__ status,
                                      int interleaved) {
    __shared__ float scratch[33];
    grid_dep_launch();
    grid_dep_wait();
    const size_t t = blockIdx.x;
    const int slot = tok_slot[t];
    if (dq) {
        float s = 0.f;
        if (slot >= 0)
            for (int i = threadIdx.x; i < q_rank; i += blockDim.x) { const float v = to_f32(dq[t * lddq + i]); s = fmaf(v, v, s); }
        const float rstd = 1.0f / sqrtf(block_sum(s, scratch) / (float)q_rank + eps);
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
            cq_out[t * ldcq + i] = from_f32<T>(slot >= 0 ? to_f32(dq[t * lddq + i]) * rstd * load_as_f32(wq, wq_dtype, i) : 0.f);
    }
    if (!dkv || slot < 0) return;
    const int pos = tok_pos[t];
    const int page = pos >= 0 ? page_table[(size_t)slot * max_pages + (pos >> page_shift)] : -1;
    if (page < 0) { if (threadIdx.x == 0) atomicExch(status, 2); return; }
    const size_t row = ((size_t)page << page_shift) + (pos & ((1 << page_shift) - 1));
    T* kdst = k_cache + row * (kv_rank + rot_dim);
    T* vdst = v_cache + row * kv_rank;
    float s = 0.f;
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) { const float v = to_f32(dkv[t * lddkv + i]); s = fmaf(v, v, s); }
    const float rstd = 1.0f / sqrtf(block_sum(s, scratch) / (float)kv_rank + eps);
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) {
        const T c = from_f32<T>(to_f32(dkv[t * lddkv + i]) * rstd * load_as_f32(wkv, wkv_dtype, i));
        kdst[i] = c;
        vdst[i] = c;
    }
    const T* kr = dkv + t * lddkv + kv_rank;
    const int half = rot_dims >> 1;
    for (int i = threadIdx.x; i < rot_dim; i += blockDim.x) {
        if (i >= rot_dims) { kdst[kv_rank + i] = kr[i]; continue; }
        const int j = interleaved ? i >> 1 : (i < half ? i : i - half);
        const bool first = interleaved ? !(i & 1) : i < half;
        double sn, cs;
        sincos((double)pos * freq[j], &sn, &cs);
        const float c = (float)cs * mag, sv = (float)sn * mag;
        const float u = to_f32(kr[interleaved ? 2 * j : j]), v = to_f32(kr[interleaved ? 2 * j + 1 : j + half]);
        kdst[kv_rank + i] = from_f32<T>(first ? u * c - v * sv : v * c + u * sv);
    }
}

// q [T, H * (dn + dr)] -> q_abs [T, H * (r + dr)]: head h's last dr elements rotated and written behind the r
// elements that the folded product fills.
template <typename T>
__global__ void latent_q_rotate_kernel(T* __restrict__ q_abs, size_t ldqa, const T* __restrict__ q, size_t ldq, int H,
                                       int dn, int dr, int r, int rot_dims, const double* __restrict__ freq, float mag,
                                       const int32_t* __restrict__ tok_slot, const int32_t* __restrict__ tok_pos,
                                       int interleaved) {
    extern __shared__ float cs_sn[];                    // the token's cosines and sines, taken once for all heads
    grid_dep_launch();
    grid_dep_wait();
    const size_t t = blockIdx.x;
    const int slot = tok_slot[t];
    const int pos = slot >= 0 ? tok_pos[t] : 0;
    const int half = rot_dims >> 1;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        double sn, cs;
        sincos((double)pos * freq[j], &sn, &cs);
        cs_sn[2 * j] = (float)cs * mag;
        cs_sn[2 * j + 1] = (float)sn * mag;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < H * dr; e += blockDim.x) {
        const int h = e / dr, i = e - h * dr;
        const T* src = q + t * ldq + (size_t)h * (dn + dr) + dn;
        T* dst = q_abs + t * ldqa + (size_t)h * (r + dr) + r;
        if (slot < 0) { dst[i] = from_f32<T>(0.f); continue; }
        if (i >= rot_dims) { dst[i] = src[i]; continue; }
        const int j = interleaved ? i >> 1 : (i < half ? i : i - half);
        const bool first = interleaved ? !(i & 1) : i < half;
        const float c = cs_sn[2 * j], sv = cs_sn[2 * j + 1];
        const float u = to_f32(src[interleaved ? 2 * j : j]), v = to_f32(src[interleaved ? 2 * j + 1 : j + half]);
        dst[i] = from_f32<T>(first ? u * c - v * sv : v * c + u * sv);
    }
}

// out[t, h, n] = sum_k x[t, h, k] * w[h][n][k]: one small matrix per head, for steps of few tokens (a product per
// head costs a launch each there).  A block takes one head, HL_N output features and up to HL_T tokens, whose rows
// it stages in shared memory as 32-bit floats; a warp takes a feature at a time, lanes along k; 32-bit sums in a
// fixed order.
constexpr int HL_T = 8, HL_N = 32;

template <typename T>
__global__ void head_linear_kernel(T* __restrict__ out, size_t ldo, size_t head_o, const T* __restrict__ x, size_t ldx,
                                   size_t head_x, const T* __restrict__ w, int n_tokens, int N, int K) {
    extern __shared__ float xs[];                       // [HL_T][K]
    grid_dep_launch();
    grid_dep_wait();
    const int h = blockIdx.x, n0 = blockIdx.y * HL_N, t0 = blockIdx.z * HL_T;
    const int nt = min(HL_T, n_tokens - t0);
    for (int e = threadIdx.x; e < nt * K; e += blockDim.x) {
        const int tt = e / K, k = e - tt * K;
        xs[e] = to_f32(x[(size_t)(t0 + tt) * ldx + (size_t)h * head_x + k]);
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    for (int n = n0 + warp; n < min(N, n0 + HL_N); n += warps) {
        const T* wr = w + ((size_t)h * N + n) * K;
        float acc[HL_T];
#pragma unroll
        for (int tt = 0; tt < HL_T; ++tt) acc[tt] = 0.f;
        for (int k = lane; k < K; k += 32) {
            const float wv = to_f32(wr[k]);
#pragma unroll
            for (int tt = 0; tt < HL_T; ++tt)
                if (tt < nt) acc[tt] = fmaf(wv, xs[tt * K + k], acc[tt]);
        }
#pragma unroll
        for (int tt = 0; tt < HL_T; ++tt) {
            const float total = warp_sum(acc[tt]);
            if (tt < nt && lane == 0) out[(size_t)(t0 + tt) * ldo + (size_t)h * head_o + n] = from_f32<T>(total);
        }
    }
}

}  // namespace

// dq [T, q_rank] (may be null: no query latent) -> cq_out; dkv [T, kv_rank + rot_dim] (null for a layer that reads
// another layer's cache) -> the cache entry's keys [pages][1][page_tokens][kv_rank + rot_dim] and values
// [pages][1][page_tokens][kv_rank].  `freq`: rot_dims / 2 doubles on the device.
QS_API int qs_latent_prepare(void* cq_out, long long ldcq, const void* dq, long long lddq, const void* wq, int wq_dtype,
                             int q_rank, const void* dkv, long long lddkv, const void* wkv, int wkv_dtype, int kv_rank,
                             int rot_dim, int rot_dims, const double* freq, float mag, float eps, int dtype,
                             const int32_t* tok_slot, const int32_t* tok_pos, const int32_t* page_table, int max_pages,
                             int page_tokens, void* k_cache, void* v_cache, int T_tokens, int32_t* status,
                             int interleaved, cudaStream_t stream) {
    if (T_tokens == 0) return QS_OK;
    QS_REQUIRE(T_tokens > 0 && (dq || dkv), "latent_prepare: nothing to do");
    QS_REQUIRE(!dq || (cq_out && wq && q_rank > 0), "latent_prepare: a query latent without its norm");
    QS_REQUIRE(!dkv || (wkv && kv_rank > 0 && rot_dim >= 0 && k_cache && v_cache && page_table && freq),
               "latent_prepare: a key latent without its norm, cache or frequencies");
    QS_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= rot_dim, "latent_prepare: %d rotated of %d dims", rot_dims, rot_dim);
    QS_REQUIRE(page_tokens > 0 && (page_tokens & (page_tokens - 1)) == 0, "latent_prepare: page size %d is no power of two", page_tokens);
    int shift = 0;
    while ((1 << shift) < page_tokens) ++shift;
    const int widest = q_rank > kv_rank ? q_rank : kv_rank;
    const int threads = widest >= 1024 ? 256 : 128;
    cudaError_t e;
#define GO(T) e = qs_launch_dependent(latent_prepare_kernel<T>, dim3(T_tokens), dim3(threads), 0, stream, (T*)cq_out, (size_t)ldcq, \
        (const T*)dq, (size_t)lddq, wq, wq_dtype, q_rank, (const T*)dkv, (size_t)lddkv, wkv, wkv_dtype, kv_rank, rot_dim, rot_dims, \
        freq, mag, eps, tok_slot, tok_pos, page_table, max_pages, shift, (T*)k_cache, (T*)v_cache, status, interleaved)
    if (dtype == QS_F32) GO(float);
    else if (dtype == QS_BF16) GO(__nv_bfloat16);
    else return qs_fail(QS_ERR_INVALID_INPUT, "latent_prepare: unknown dtype %d", dtype);
#undef GO
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "latent_prepare: %s", cudaGetErrorString(e));
    return qs_check_launch("latent_prepare");
}

QS_API int qs_latent_q_rotate(void* q_abs, long long ldqa, const void* q, long long ldq, int dtype, int H, int dn, int dr,
                              int r, int rot_dims, const double* freq, float mag, const int32_t* tok_slot,
                              const int32_t* tok_pos, int T_tokens, int interleaved, cudaStream_t stream) {
    if (T_tokens == 0 || dr == 0) return QS_OK;
    QS_REQUIRE(T_tokens > 0 && H > 0 && dn >= 0 && dr > 0 && r > 0 && freq, "latent_q_rotate: bad sizes");
    QS_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dr, "latent_q_rotate: %d rotated of %d dims", rot_dims, dr);
    const int threads = H * dr >= 1024 ? 256 : 128;
    cudaError_t e;
#define GO(T) e = qs_launch_dependent(latent_q_rotate_kernel<T>, dim3(T_tokens), dim3(threads), (size_t)(rot_dims > 0 ? rot_dims : 1) * sizeof(float), stream, (T*)q_abs, (size_t)ldqa, \
        (const T*)q, (size_t)ldq, H, dn, dr, r, rot_dims, freq, mag, tok_slot, tok_pos, interleaved)
    if (dtype == QS_F32) GO(float);
    else if (dtype == QS_BF16) GO(__nv_bfloat16);
    else return qs_fail(QS_ERR_INVALID_INPUT, "latent_q_rotate: unknown dtype %d", dtype);
#undef GO
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "latent_q_rotate: %s", cudaGetErrorString(e));
    return qs_check_launch("latent_q_rotate");
}

// x: head h's K inputs of token t at x[t * ldx + h * head_x + k]; w [H][N][K] contiguous; out likewise with ldo, head_o.
QS_API int qs_head_linear(void* out, long long ldo, long long head_o, const void* x, long long ldx, long long head_x,
                          const void* w, int dtype, int T_tokens, int H, int N, int K, cudaStream_t stream) {
    if (T_tokens == 0) return QS_OK;
    QS_REQUIRE(T_tokens > 0 && H > 0 && N > 0 && K > 0 && H <= 65535, "head_linear: bad sizes");
    const size_t smem = (size_t)HL_T * K * sizeof(float);
    QS_REQUIRE(smem <= 200 * 1024, "head_linear: %d inputs per head do not fit shared memory", K);
    dim3 grid(H, (N + HL_N - 1) / HL_N, (T_tokens + HL_T - 1) / HL_T);
    cudaError_t e = cudaSuccess;
#define GO(T) do { if (smem > 48 * 1024) e = cudaFuncSetAttribute(head_linear_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    if (e == cudaSuccess) e = qs_launch_dependent(head_linear_kernel<T>, grid, dim3(256), smem, stream, (T*)out, (size_t)ldo, (size_t)head_o, \
        (const T*)x, (size_t)ldx, (size_t)head_x, (const T*)w, T_tokens, N, K); } while (0)
    if (dtype == QS_F32) GO(float);
    else if (dtype == QS_BF16) GO(__nv_bfloat16);
    else return qs_fail(QS_ERR_INVALID_INPUT, "head_linear: unknown dtype %d", dtype);
#undef GO
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "head_linear: %s", cudaGetErrorString(e));
    return qs_check_launch("head_linear");
}
