// What a gated delta rule needs between its projections and its scan.
//
// q, k (G heads of dk) and v (H heads of dv) each pass a short causal convolution over time per channel
// (taps [channels, n]: tap n - 1 weighs the token itself, tap n - 1 - j the token j places back, and what lies before a
// sequence counts as zero) and silu; q and k then become unit vectors per head, x / sqrt(sum x^2 + unit_eps), q also
// times q_scale.  The decay per token, head
// and key channel is g = exp(-exp(A_log_h) * softplus(a)), the step size per token and head beta = sigmoid(b).
// Everything is 32-bit and leaves in 32-bit: these values enter the recurrence.
//
// The convolution's last n - 1 inputs of a sequence are state: [slots][n - 1][C] in the inputs' type, channels in
// the order q | k | v, row n - 2 the newest, zero when the slot is taken.  `delta_prepare_kernel` reads it for the
// tokens whose predecessors came in earlier steps; `conv_state_update_kernel` runs after it and leaves the last
// n - 1 inputs of what the slot held and the step brought.
#include "common.cuh"

namespace {

constexpr int MAX_TAPS = 8;

__device__ __forceinline__ float softplus_f32(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

template <typename TI>
__global__ void delta_prepare_kernel(float* __restrict__ qo, float* __restrict__ ko, float* __restrict__ vo,
                                     float* __restrict__ go, float* __restrict__ bo,
                                     const TI* __restrict__ q, const TI* __restrict__ k, const TI* __restrict__ v, size_t ldp,
                                     const void* __restrict__ wq, const void* __restrict__ wk, const void* __restrict__ wv,
                                     int w_dtype, int taps, const TI* __restrict__ conv_state, size_t slot_stride,
                                     const float* __restrict__ a, size_t lda, const float* __restrict__ bl, size_t ldb,
                                     const void* __restrict__ a_log, int a_log_dtype,
                                     const int32_t* __restrict__ tok_slot, const int32_t* __restrict__ tok_pos,
                                     int G, int H, int dk, int dv, float q_scale, float unit_eps) {
    extern __shared__ float x_of[];                     // [C] the token's channels after convolution and silu
    __shared__ float inv_norm[64];                      // per head of q and k, in rounds of 64
    grid_dep_launch();
    grid_dep_wait();
    const int t = blockIdx.x;
    const int nq = G * dk, nv = H * dv, C = 2 * nq + nv;
    const int slot = tok_slot[t];
    if (slot < 0) {                                     // a row that belongs to nobody
        for (int c = threadIdx.x; c < nq; c += blockDim.x) { qo[(size_t)t * nq + c] = 0.f; ko[(size_t)t * nq + c] = 0.f; }
        for (int c = threadIdx.x; c < nv; c += blockDim.x) vo[(size_t)t * nv + c] = 0.f;
        for (int c = threadIdx.x; c < H * dk; c += blockDim.x) go[(size_t)t * H * dk + c] = 1.f;
        for (int c = threadIdx.x; c < H; c += blockDim.x) bo[(size_t)t * H + c] = 0.f;
        return;
    }
    const int pos = tok_pos[t];
    // how many of the token's predecessors came with this step (they lie in the rows just above), up to taps - 1
    int here = 0;
    while (here < taps - 1 && t - here - 1 >= 0 && tok_slot[t - here - 1] == slot && tok_pos[t - here - 1] == pos - here - 1) ++here;
    const TI* held = conv_state + (size_t)slot * slot_stride;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const TI* src; const void* w; int ch;
        if (c < nq) { src = q; w = wq; ch = c; }
        else if (c < 2 * nq) { src = k; w = wk; ch = c - nq; }
        else { src = v; w = wv; ch = c - 2 * nq; }
        float acc = 0.f;
        for (int j = 0; j < taps; ++j) {                // the input j tokens back meets tap number taps - 1 - j
            float x;
            if (j <= here) x = to_f32(src[(size_t)(t - j) * ldp + ch]);
            else x = to_f32(held[(size_t)(taps - 1 - (j - here)) * C + c]);
            acc = fmaf(load_as_f32(w, w_dtype, (size_t)ch * taps + taps - 1 - j), x, acc);
        }
        x_of[c] = silu_f32(acc);
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int first = 0; first < 2 * G; first += 64) {   // the heads of q, then those of k
        const int n = min(64, 2 * G - first);
        for (int hd = warp; hd < n; hd += warps) {
            const float* x = x_of + (size_t)(first + hd) * dk;
            float sq = 0.f;
            for (int i = lane; i < dk; i += 32) sq = fmaf(x[i], x[i], sq);
            sq = warp_sum(sq);
            if (lane == 0) inv_norm[hd] = 1.0f / sqrtf(sq + unit_eps);
        }
        __syncthreads();
        for (int e = threadIdx.x; e < n * dk; e += blockDim.x) {
            const int hd = first + e / dk, i = e % dk;
            const float val = x_of[(size_t)hd * dk + i] * inv_norm[e / dk];
            if (hd < G) qo[(size_t)t * nq + (size_t)hd * dk + i] = val * q_scale;
            else ko[(size_t)t * nq + (size_t)(hd - G) * dk + i] = val;
        }
        __syncthreads();
    }
    for (int c = threadIdx.x; c < nv; c += blockDim.x) vo[(size_t)t * nv + c] = x_of[2 * nq + c];
    for (int c = threadIdx.x; c < H * dk; c += blockDim.x) {
        const float rate = expf(load_as_f32(a_log, a_log_dtype, c / dk));
        go[(size_t)t * H * dk + c] = expf(-rate * softplus_f32(a[(size_t)t * lda + c]));
    }
    for (int c = threadIdx.x; c < H; c += blockDim.x) bo[(size_t)t * H + c] = sigmoid_f32(bl[(size_t)t * ldb + c]);
}

template <typename TI>
__global__ void conv_state_update_kernel(TI* __restrict__ conv_state, size_t slot_stride, const TI* __restrict__ q,
                                         const TI* __restrict__ k, const TI* __restrict__ v, size_t ldp, int nq, int nv,
                                         int taps, const int32_t* __restrict__ seq_start,
                                         const int32_t* __restrict__ seq_slot) {
    grid_dep_launch();
    grid_dep_wait();
    const int s = blockIdx.x;
    const int slot = seq_slot[s];
    const int t0 = seq_start[s], n = seq_start[s + 1] - t0;
    if (slot < 0 || n <= 0) return;
    const int C = 2 * nq + nv, keep = taps - 1;
    TI* held = conv_state + (size_t)slot * slot_stride;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        const TI* src; int ch;
        if (c < nq) { src = q; ch = c; }
        else if (c < 2 * nq) { src = k; ch = c - nq; }
        else { src = v; ch = c - 2 * nq; }
        // row j of the new state is the input n - keep + j rows into the step, or, before the step, what row j + n
        // held: rows are taken in rising order, so a row is read before this thread overwrites it
        for (int j = 0; j < keep; ++j) {
            const int idx = n - keep + j;
            held[(size_t)j * C + c] = idx >= 0 ? src[(size_t)(t0 + idx) * ldp + ch] : held[(size_t)(j + n) * C + c];
        }
    }
}

}  // namespace

// q, k, v: three column ranges of one product's result (row stride ldp, type `dtype`); a [T, H * dk] and bl [T, H]
// float32; conv_state [slots][taps - 1][2 G dk + H dv] of type `dtype`.  Outputs float32, contiguous rows.
QS_API int qs_delta_prepare(float* qo, float* ko, float* vo, float* go, float* bo, const void* q, const void* k, const void* v,
                            long long ldp, int dtype, const void* wq, const void* wk, const void* wv, int w_dtype, int taps,
                            const void* conv_state, long long slot_stride, const float* a, long long lda, const float* bl,
                            long long ldb, const void* a_log, int a_log_dtype, const int32_t* tok_slot,
                            const int32_t* tok_pos, int T_rows, int G, int H, int dk, int dv, float q_scale, float unit_eps,
                            cudaStream_t stream) {
    if (T_rows == 0) return QS_OK;
    QS_REQUIRE(T_rows > 0 && G > 0 && H > 0 && dk > 0 && dv > 0, "delta_prepare: bad sizes");
    QS_REQUIRE(taps >= 1 && taps <= MAX_TAPS, "delta_prepare: %d taps (1 to %d)", taps, MAX_TAPS);
    QS_REQUIRE(taps == 1 || conv_state, "delta_prepare: a convolution without its state");
    const size_t smem = (size_t)(2 * G * dk + H * dv) * sizeof(float);
    QS_REQUIRE(smem <= 200 * 1024, "delta_prepare: %d channels above the shared memory of a block", 2 * G * dk + H * dv);
    const int threads = 256;
    cudaError_t e;
#define GO(TI) do { e = smem > 48 * 1024 ? cudaFuncSetAttribute(delta_prepare_kernel<TI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) \
                                          : cudaSuccess; \
    if (e == cudaSuccess) e = qs_launch_dependent(delta_prepare_kernel<TI>, dim3(T_rows), dim3(threads), smem, stream, qo, ko, vo, go, bo, \
        (const TI*)q, (const TI*)k, (const TI*)v, (size_t)ldp, wq, wk, wv, w_dtype, taps, (const TI*)conv_state, (size_t)slot_stride, \
        a, (size_t)lda, bl, (size_t)ldb, a_log, a_log_dtype, tok_slot, tok_pos, G, H, dk, dv, q_scale, unit_eps); } while (0)
    if (dtype == QS_F32) GO(float);
    else if (dtype == QS_BF16) GO(__nv_bfloat16);
    else return qs_fail(QS_ERR_INVALID_INPUT, "delta_prepare: unknown dtype %d", dtype);
#undef GO
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "delta_prepare: %s", cudaGetErrorString(e));
    return qs_check_launch("delta_prepare");
}

QS_API int qs_conv_state_update(void* conv_state, long long slot_stride, const void* q, const void* k, const void* v,
                                long long ldp, int dtype, int nq, int nv, int taps, const int32_t* seq_start,
                                const int32_t* seq_slot, int n_seq, cudaStream_t stream) {
    if (n_seq == 0 || taps <= 1) return QS_OK;
    QS_REQUIRE(n_seq > 0 && nq > 0 && nv > 0 && taps <= MAX_TAPS, "conv_state_update: bad sizes");
    const int C = 2 * nq + nv, threads = 256;
    dim3 grid(n_seq, (C + threads - 1) / threads);
    cudaError_t e;
    if (dtype == QS_F32)
        e = qs_launch_dependent(conv_state_update_kernel<float>, grid, dim3(threads), 0, stream, (float*)conv_state,
                                (size_t)slot_stride, (const float*)q, (const float*)k, (const float*)v, (size_t)ldp, nq, nv, taps,
                                seq_start, seq_slot);
    else if (dtype == QS_BF16)
        e = qs_launch_dependent(conv_state_update_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream,
                                (__nv_bfloat16*)conv_state, (size_t)slot_stride, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k,
                                (const __nv_bfloat16*)v, (size_t)ldp, nq, nv, taps, seq_start, seq_slot);
    else return qs_fail(QS_ERR_INVALID_INPUT, "conv_state_update: unknown dtype %d", dtype);
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "conv_state_update: %s", cudaGetErrorString(e));
    return qs_check_launch("conv_state_update");
}
