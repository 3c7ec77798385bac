// RMS norms and the small kernels around a residual stream that is kept in 32-bit:
//
//   rmsnorm            y = x / sqrt(mean(x^2) + eps) * (offset + w)
//   residual_rmsnorm   x <- x + mult * y (32-bit, in place), and optionally h = rmsnorm(x) in the same pass
//   branch_norm        x <- x + norm_b(y) * w_b (in place), and optionally h = norm(x) * w in the same pass, with
//                      norm = layer norm without bias or RMS norm: layers that norm a branch before they add it
//   gated_group_norm   out = o / sqrt(mean_group(o^2) + eps) * w * act(gate), groups of consecutive elements
//                      (one group = the whole row, or one per head; group 0 = no norm, only the gate)
//   gated_act          out = act(a) * b for the two halves [a | b] of a fused projection (gated feed-forward)
//   activate           x <- act(x) in place
//   embedding_hashed   x = table[token] * scale + pair_table[hash(previous token, token)]
//   keep_last_rows     state[slot] = the last row each sequence brought in this step
//
// Every sum is taken in 32-bit in a fixed order (block_sum / warp_sum), whatever the storage types.
#include "common.cuh"

namespace {

// ----------------------------------------------------------------------------- rmsnorm

// One block per row, the row in shared memory as 32-bit floats.  With `y` the row is first updated:
// x <- x + mult * y, written back to `x_out` (which may be x itself).  `h_out` may be null (update only).
template <typename TX, typename TY, typename TH>
__global__ void residual_rmsnorm_kernel(TH* __restrict__ h_out, size_t ldh, TX* x_out, const TX* x, size_t ldx,
                                        const TY* __restrict__ y, size_t ldy, float mult,
                                        const void* __restrict__ w, int w_dtype, float offset, int D, float eps) {
    extern __shared__ float row[];
    __shared__ float scratch[33];
    grid_dep_launch();
    grid_dep_wait();
    const TX* src = x + (size_t)blockIdx.x * ldx;
    float s = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        float v = to_f32(src[i]);
        if (y) {
            v = fmaf(mult, to_f32(y[(size_t)blockIdx.x * ldy + i]), v);
            x_out[(size_t)blockIdx.x * ldx + i] = from_f32<TX>(v);
        }
        row[i] = v;
        s = fmaf(v, v, s);
    }
    if (!h_out) return;
    const float rstd = 1.0f / sqrtf(block_sum(s, scratch) / (float)D + eps);
    TH* dst = h_out + (size_t)blockIdx.x * ldh;
    for (int i = threadIdx.x; i < D; i += blockDim.x)
        dst[i] = from_f32<TH>(row[i] * rstd * (offset + load_as_f32(w, w_dtype, i)));
}

template <typename TX, typename TY, typename TH>
int launch_norm(void* h_out, long long ldh, void* x_out, const void* x, long long ldx, const void* y, long long ldy,
                float mult, const void* w, int w_dtype, float offset, int rows, int D, float eps, cudaStream_t stream) {
    const size_t smem = (size_t)D * sizeof(float);
    const int threads = D >= 4096 ? 512 : (D >= 1024 ? 256 : 128);
    auto kernel = residual_rmsnorm_kernel<TX, TY, TH>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "rmsnorm: %s", cudaGetErrorString(e));
    }
    cudaError_t e = qs_launch_dependent(kernel, dim3(rows), dim3(threads), smem, stream, (TH*)h_out, (size_t)ldh,
                                        (TX*)x_out, (const TX*)x, (size_t)ldx, (const TY*)y, (size_t)ldy, mult, w, w_dtype,
                                        offset, D, eps);
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "rmsnorm: %s", cudaGetErrorString(e));
    return qs_check_launch("rmsnorm");
}

// ----------------------------------------------------------------------------- norms around a branch

// One block per row, the row in shared memory as 32-bit floats.  The statistic of `v` over the row: with `center`
// mean and variance of the deviations (layer norm), without it the mean square (RMS norm); returns (mean, rstd).
__device__ __forceinline__ float2 row_statistic(const float* row, int D, float eps, int center, float* scratch) {
    float mean = 0.f;
    if (center) {
        float s = 0.f;
        for (int i = threadIdx.x; i < D; i += blockDim.x) s += row[i];
        mean = block_sum(s, scratch) / (float)D;
    }
    float q = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) { const float d = row[i] - mean; q = fmaf(d, d, q); }
    const float var = block_sum(q, scratch) / (float)D;
    return make_float2(mean, 1.0f / sqrtf(var + eps));
}

// With y: x <- x + norm(y) * wy (wy null: x + y), written back in x's type.  With h_out: h = norm(x) * w, or, without
// w, x itself in h's type (a sublayer that reads the stream as it is).
// h_out may be x itself (a norm in place).  A thread reads back only what it wrote to `row`.
template <typename TX, typename TY, typename TH>
__global__ void branch_norm_kernel(TH* h_out, size_t ldh, TX* x, size_t ldx, const TY* __restrict__ y, size_t ldy,
                                   const void* __restrict__ wy, int wy_dtype, const void* __restrict__ w, int w_dtype,
                                   int D, float eps, int center) {
    extern __shared__ float row[];
    __shared__ float scratch[33];
    grid_dep_launch();
    grid_dep_wait();
    TX* xr = x + (size_t)blockIdx.x * ldx;
    if (y) {
        for (int i = threadIdx.x; i < D; i += blockDim.x) row[i] = to_f32(y[(size_t)blockIdx.x * ldy + i]);
        float2 st = make_float2(0.f, 1.f);
        if (wy) st = row_statistic(row, D, eps, center, scratch);
        for (int i = threadIdx.x; i < D; i += blockDim.x) {
            const float b = wy ? (row[i] - st.x) * st.y * load_as_f32(wy, wy_dtype, i) : row[i];
            const float v = to_f32(xr[i]) + b;
            xr[i] = from_f32<TX>(v);
            row[i] = v;
        }
    } else {
        for (int i = threadIdx.x; i < D; i += blockDim.x) row[i] = to_f32(xr[i]);
    }
    if (!h_out) return;
    TH* dst = h_out + (size_t)blockIdx.x * ldh;
    if (!w) {
        for (int i = threadIdx.x; i < D; i += blockDim.x) dst[i] = from_f32<TH>(row[i]);
        return;
    }
    const float2 st = row_statistic(row, D, eps, center, scratch);
    for (int i = threadIdx.x; i < D; i += blockDim.x)
        dst[i] = from_f32<TH>((row[i] - st.x) * st.y * load_as_f32(w, w_dtype, i));
}

template <typename TX, typename TY, typename TH>
int launch_branch_norm(void* h_out, long long ldh, void* x, long long ldx, const void* y, long long ldy, const void* wy,
                       int wy_dtype, const void* w, int w_dtype, int rows, int D, float eps, int center, cudaStream_t stream) {
    const size_t smem = (size_t)D * sizeof(float);
    const int threads = D >= 4096 ? 512 : (D >= 1024 ? 256 : 128);
    auto kernel = branch_norm_kernel<TX, TY, TH>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "branch_norm: %s", cudaGetErrorString(e));
    }
    cudaError_t e = qs_launch_dependent(kernel, dim3(rows), dim3(threads), smem, stream, (TH*)h_out, (size_t)ldh, (TX*)x,
                                        (size_t)ldx, (const TY*)y, (size_t)ldy, wy, wy_dtype, w, w_dtype, D, eps, center);
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "branch_norm: %s", cudaGetErrorString(e));
    return qs_check_launch("branch_norm");
}

// ----------------------------------------------------------------------------- gated group norm

// One block per row.  group == n: one norm over the row (block sum).  0 < group < n: a warp per group, groups dealt
// to the warps in turn.  group == 0: no norm.  Then * w[c] (if given) * act(gate[c / gate_span]) (if given; a span
// above 1 is one gate value for that many neighbouring elements, a head's say).
template <typename TI, typename TG, typename TO>
__global__ void gated_group_norm_kernel(TO* __restrict__ out, size_t ldo, const TI* __restrict__ o, size_t ldi,
                                        const void* __restrict__ w, int w_dtype, const TG* __restrict__ gate, size_t ldg,
                                        int gate_act, int n, int group, float eps, int gate_span) {
    extern __shared__ float rstd_of[];               // one per group (at least one)
    __shared__ float scratch[33];
    grid_dep_launch();
    grid_dep_wait();
    const TI* src = o + (size_t)blockIdx.x * ldi;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    if (group == n) {
        float s = 0.f;
        for (int i = threadIdx.x; i < n; i += blockDim.x) { const float v = to_f32(src[i]); s = fmaf(v, v, s); }
        const float total = block_sum(s, scratch);
        if (threadIdx.x == 0) rstd_of[0] = 1.0f / sqrtf(total / (float)n + eps);
    } else if (group > 0) {
        for (int g = warp; g * group < n; g += warps) {
            float s = 0.f;
            for (int i = lane; i < group; i += 32) { const float v = to_f32(src[g * group + i]); s = fmaf(v, v, s); }
            s = warp_sum(s);
            if (lane == 0) rstd_of[g] = 1.0f / sqrtf(s / (float)group + eps);
        }
    }
    __syncthreads();
    TO* dst = out + (size_t)blockIdx.x * ldo;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float v = to_f32(src[i]);
        if (group > 0) v *= rstd_of[i / group];
        if (w) v *= load_as_f32(w, w_dtype, i);
        if (gate) v *= apply_activation(to_f32(gate[(size_t)blockIdx.x * ldg + (gate_span > 1 ? i / gate_span : i)]), gate_act);
        dst[i] = from_f32<TO>(v);
    }
}

template <typename TI, typename TG, typename TO>
int launch_gated(void* out, long long ldo, const void* o, long long ldi, const void* w, int w_dtype, const void* gate,
                 long long ldg, int gate_act, int rows, int n, int group, float eps, int gate_span, cudaStream_t stream) {
    const int n_groups = group > 0 ? n / group : 1;
    const int threads = n >= 2048 ? 256 : 128;
    cudaError_t e = qs_launch_dependent(gated_group_norm_kernel<TI, TG, TO>, dim3(rows), dim3(threads),
                                        (size_t)n_groups * sizeof(float), stream, (TO*)out, (size_t)ldo, (const TI*)o,
                                        (size_t)ldi, w, w_dtype, (const TG*)gate, (size_t)ldg, gate_act, n, group, eps, gate_span);
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "gated_group_norm: %s", cudaGetErrorString(e));
    return qs_check_launch("gated_group_norm");
}

// ----------------------------------------------------------------------------- gated activation

// One row per blockIdx.x, a block of columns per blockIdx.y.  VEC (bfloat16, F a multiple of 8, 16-byte aligned
// rows): eight columns per thread as one 16-byte piece of each half.
template <typename T, bool VEC>
__global__ void gated_act_kernel(T* __restrict__ out, size_t ldo, const T* __restrict__ ab, size_t ldi, int F, int act) {
    grid_dep_launch();
    grid_dep_wait();
    const size_t r = blockIdx.x;
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * (VEC ? 8 : 1);
    if (c >= F) return;
    if (VEC) {
        const uint4 a = *reinterpret_cast<const uint4*>(ab + r * ldi + c), b = *reinterpret_cast<const uint4*>(ab + r * ldi + F + c);
        const uint32_t au[4] = {a.x, a.y, a.z, a.w}, bu[4] = {b.x, b.y, b.z, b.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float a0 = __uint_as_float(au[j] << 16), a1 = __uint_as_float(au[j] & 0xffff0000u);
            const float b0 = __uint_as_float(bu[j] << 16), b1 = __uint_as_float(bu[j] & 0xffff0000u);
            const __nv_bfloat162 p = __floats2bfloat162_rn(apply_activation(a0, act) * b0, apply_activation(a1, act) * b1);
            o[j] = *reinterpret_cast<const uint32_t*>(&p);
        }
        *reinterpret_cast<uint4*>(out + r * ldo + c) = make_uint4(o[0], o[1], o[2], o[3]);
    } else {
        const float a = to_f32(ab[r * ldi + c]), b = to_f32(ab[r * ldi + F + c]);
        out[r * ldo + c] = from_f32<T>(apply_activation(a, act) * b);
    }
}

// The clamped gated unit of two halves [a | b]: g = min(a, limit), u = clamp(b, -limit, limit),
// out = g * sigmoid(alpha * g) * (u + shift); 32-bit arithmetic, rounded once.  limit <= 0: no clamp.
__device__ __forceinline__ float clamped_glu(float g, float u, float limit, float alpha, float shift) {
    if (limit > 0.f) { g = fminf(g, limit); u = fminf(fmaxf(u, -limit), limit); }
    return g * sigmoid_f32(alpha * g) * (u + shift);
}

// VEC (bfloat16, F a multiple of 8, 16-byte aligned rows): eight columns per thread as one 16-byte piece of each half.
template <typename T, bool VEC>
__global__ void clamped_glu_kernel(T* __restrict__ out, size_t ldo, const T* __restrict__ ab, size_t ldi, int F, float limit,
                                   float alpha, float shift) {
    grid_dep_launch();
    grid_dep_wait();
    const size_t r = blockIdx.x;
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * (VEC ? 8 : 1);
    if (c >= F) return;
    if (VEC) {
        const uint4 a = *reinterpret_cast<const uint4*>(ab + r * ldi + c), b = *reinterpret_cast<const uint4*>(ab + r * ldi + F + c);
        const uint32_t au[4] = {a.x, a.y, a.z, a.w}, bu[4] = {b.x, b.y, b.z, b.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float a0 = __uint_as_float(au[j] << 16), a1 = __uint_as_float(au[j] & 0xffff0000u);
            const float b0 = __uint_as_float(bu[j] << 16), b1 = __uint_as_float(bu[j] & 0xffff0000u);
            const __nv_bfloat162 p = __floats2bfloat162_rn(clamped_glu(a0, b0, limit, alpha, shift), clamped_glu(a1, b1, limit, alpha, shift));
            o[j] = *reinterpret_cast<const uint32_t*>(&p);
        }
        *reinterpret_cast<uint4*>(out + r * ldo + c) = make_uint4(o[0], o[1], o[2], o[3]);
    } else {
        out[r * ldo + c] = from_f32<T>(clamped_glu(to_f32(ab[r * ldi + c]), to_f32(ab[r * ldi + F + c]), limit, alpha, shift));
    }
}

// x <- act(x), in 32-bit, rounded once: for activations that the matrix products' epilogues do not offer.
template <typename T>
__global__ void activate_kernel(T* __restrict__ x, size_t ld, int n, int act) {
    grid_dep_launch();
    grid_dep_wait();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c < n) x[(size_t)blockIdx.x * ld + c] = from_f32<T>(apply_activation_wide(to_f32(x[(size_t)blockIdx.x * ld + c]), act));
}

// ----------------------------------------------------------------------------- hashed-pair embedding

// x[t] = table[token] * scale + pair[row], row = (previous * mul_prev + token * mul_cur) mod buckets, and row
// `buckets` for a sequence's first token.  The previous token is the row above if it belongs to the same
// sequence, else what the sequence's earlier steps left in `last_token[slot]`.
template <typename TO, typename TT>
__global__ void embedding_hashed_kernel(TO* __restrict__ out, const TT* __restrict__ table, float scale,
                                        const TT* __restrict__ pair, long long buckets, long long mul_prev,
                                        long long mul_cur, const int32_t* __restrict__ tokens,
                                        const int32_t* __restrict__ tok_slot, const int32_t* __restrict__ tok_pos,
                                        const int32_t* __restrict__ last_token, size_t ld_last, int D, int V) {
    const int t = blockIdx.x;
    TO* dst = out + (size_t)t * D;
    const int slot = tok_slot[t];
    if (slot < 0) {
        for (int i = threadIdx.x; i < D; i += blockDim.x) dst[i] = from_f32<TO>(0.f);
        return;
    }
    int id = tokens[t];
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);
    const TT* row = table + (size_t)id * D;
    const TT* prow = nullptr;
    if (pair) {
        long long r = buckets;
        if (tok_pos[t] > 0) {
            int prev = (t > 0 && tok_slot[t - 1] == slot) ? tokens[t - 1] : last_token[(size_t)slot * ld_last];
            prev = prev < 0 ? 0 : (prev >= V ? V - 1 : prev);
            r = ((long long)prev * mul_prev + (long long)id * mul_cur) % buckets;
            if (r < 0) r += buckets;
        }
        prow = pair + (size_t)r * D;
    }
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        float v = to_f32(row[i]) * scale;
        if (prow) v += to_f32(prow[i]);
        dst[i] = from_f32<TO>(v);
    }
}

// ----------------------------------------------------------------------------- keep last rows

// dst[slot] = the last row that each sequence of the step brought (rows of `row_bytes` bytes, 4-byte words).
__global__ void keep_last_rows_kernel(uint32_t* __restrict__ dst, size_t dst_words, const uint32_t* __restrict__ src,
                                      size_t src_words, int row_words, const int32_t* __restrict__ seq_start,
                                      const int32_t* __restrict__ seq_slot) {
    const int s = blockIdx.x;
    const int slot = seq_slot[s];
    const int a = seq_start[s], b = seq_start[s + 1];
    if (slot < 0 || b <= a) return;
    const uint32_t* from = src + (size_t)(b - 1) * src_words;
    uint32_t* to = dst + (size_t)slot * dst_words;
    for (int i = threadIdx.x; i < row_words; i += blockDim.x) to[i] = from[i];
}

}  // namespace

// h = rmsnorm(x) (y == null), or x_out = x + mult * y and h = rmsnorm(x_out) (h_out may then be null).
QS_API int qs_residual_rmsnorm(void* h_out, int h_dtype, long long ldh, void* x_out, const void* x, int x_dtype,
                               long long ldx, const void* y, int y_dtype, long long ldy, float mult, const void* w,
                               int w_dtype, float offset, int rows, int D, float eps, cudaStream_t stream) {
    if (rows == 0) return QS_OK;
    QS_REQUIRE(rows > 0 && D > 0, "rmsnorm: bad sizes rows=%d D=%d", rows, D);
    QS_REQUIRE(h_out || y, "rmsnorm: nothing to do");
    QS_REQUIRE(!h_out || w, "rmsnorm: a norm without a weight");
    QS_REQUIRE(!y || x_out, "rmsnorm: an update with nowhere to go");
    QS_REQUIRE((size_t)D * sizeof(float) <= 200 * 1024, "rmsnorm: width %d does not fit one block's shared memory", D);
    typedef __nv_bfloat16 bf16;
#define GO(TX, TY, TH) return launch_norm<TX, TY, TH>(h_out, ldh, x_out, x, ldx, y, ldy, mult, w, w_dtype, offset, rows, D, eps, stream)
    if (!y) y_dtype = x_dtype;
    if (!h_out) h_dtype = x_dtype;
    if (x_dtype == QS_F32 && y_dtype == QS_F32 && h_dtype == QS_F32) GO(float, float, float);
    if (x_dtype == QS_F32 && y_dtype == QS_F32 && h_dtype == QS_BF16) GO(float, float, bf16);
    if (x_dtype == QS_F32 && y_dtype == QS_BF16 && h_dtype == QS_BF16) GO(float, bf16, bf16);
    if (x_dtype == QS_F32 && y_dtype == QS_BF16 && h_dtype == QS_F32) GO(float, bf16, float);
    if (x_dtype == QS_BF16 && y_dtype == QS_BF16 && h_dtype == QS_BF16) GO(bf16, bf16, bf16);
#undef GO
    return qs_fail(QS_ERR_INVALID_INPUT, "rmsnorm: unsupported types x=%d y=%d h=%d", x_dtype, y_dtype, h_dtype);
}

// x <- x + norm(y) * wy (y given; wy null: plain sum) and h = norm(x) * w (h_out given; it may be x itself);
// `center` != 0: layer norm without bias, 0: RMS norm; statistics in 32-bit, eps inside the root.
QS_API int qs_branch_norm(void* h_out, int h_dtype, long long ldh, void* x, int x_dtype, long long ldx, const void* y,
                          int y_dtype, long long ldy, const void* wy, int wy_dtype, const void* w, int w_dtype, int rows,
                          int D, float eps, int center, cudaStream_t stream) {
    if (rows == 0) return QS_OK;
    QS_REQUIRE(rows > 0 && D > 0, "branch_norm: bad sizes rows=%d D=%d", rows, D);
    QS_REQUIRE(h_out || y, "branch_norm: nothing to do");
    QS_REQUIRE((size_t)D * sizeof(float) <= 200 * 1024, "branch_norm: width %d does not fit one block's shared memory", D);
    typedef __nv_bfloat16 bf16;
    if (!y) y_dtype = x_dtype;
    if (!h_out) h_dtype = x_dtype;
#define GO(TX, TY, TH) return launch_branch_norm<TX, TY, TH>(h_out, ldh, x, ldx, y, ldy, wy, wy_dtype, w, w_dtype, rows, D, eps, center, stream)
    if (x_dtype == QS_F32 && y_dtype == QS_F32 && h_dtype == QS_F32) GO(float, float, float);
    if (x_dtype == QS_F32 && y_dtype == QS_F32 && h_dtype == QS_BF16) GO(float, float, bf16);
    if (x_dtype == QS_F32 && y_dtype == QS_BF16 && h_dtype == QS_BF16) GO(float, bf16, bf16);
    if (x_dtype == QS_F32 && y_dtype == QS_BF16 && h_dtype == QS_F32) GO(float, bf16, float);
    if (x_dtype == QS_BF16 && y_dtype == QS_BF16 && h_dtype == QS_BF16) GO(bf16, bf16, bf16);
#undef GO
    return qs_fail(QS_ERR_INVALID_INPUT, "branch_norm: unsupported types x=%d y=%d h=%d", x_dtype, y_dtype, h_dtype);
}

QS_API int qs_gated_group_norm(void* out, int out_dtype, long long ldo, const void* o, int o_dtype, long long ldi,
                               const void* w, int w_dtype, const void* gate, int gate_dtype, long long ldg,
                               int gate_act, int rows, int n, int group, float eps, int gate_span, cudaStream_t stream) {
    if (rows == 0) return QS_OK;
    QS_REQUIRE(rows > 0 && n > 0 && group >= 0 && (group == 0 || n % group == 0),
               "gated_group_norm: bad sizes rows=%d n=%d group=%d", rows, n, group);
    QS_REQUIRE(gate_span >= 1 && n % gate_span == 0, "gated_group_norm: %d elements in spans of %d", n, gate_span);
    typedef __nv_bfloat16 bf16;
    if (!gate) gate_dtype = out_dtype;
#define GO(TI, TG, TO) return launch_gated<TI, TG, TO>(out, ldo, o, ldi, w, w_dtype, gate, ldg, gate_act, rows, n, group, eps, gate_span, stream)
    if (o_dtype == QS_F32 && gate_dtype == QS_F32 && out_dtype == QS_F32) GO(float, float, float);
    if (o_dtype == QS_F32 && gate_dtype == QS_BF16 && out_dtype == QS_BF16) GO(float, bf16, bf16);
    if (o_dtype == QS_F32 && gate_dtype == QS_F32 && out_dtype == QS_BF16) GO(float, float, bf16);
    if (o_dtype == QS_BF16 && gate_dtype == QS_BF16 && out_dtype == QS_BF16) GO(bf16, bf16, bf16);
#undef GO
    return qs_fail(QS_ERR_INVALID_INPUT, "gated_group_norm: unsupported types o=%d gate=%d out=%d", o_dtype, gate_dtype, out_dtype);
}

QS_API int qs_gated_act(void* out, long long ldo, const void* ab, long long ldi, int dtype, int rows, int F, int act,
                        cudaStream_t stream) {
    if (rows == 0) return QS_OK;
    QS_REQUIRE(rows > 0 && F > 0 && ldi >= 2 * (long long)F && ldo >= F, "gated_act: bad sizes rows=%d F=%d", rows, F);
    typedef __nv_bfloat16 bf16;
    cudaError_t e;
    if (dtype == QS_BF16 && F % 8 == 0 && ldi % 8 == 0 && ldo % 8 == 0 && ((uintptr_t)ab % 16) == 0 && ((uintptr_t)out % 16) == 0) {
        const int threads = F >= 2048 ? 256 : 64;
        const int by = (F / 8 + threads - 1) / threads;
        QS_REQUIRE(by <= 65535, "gated_act: %d columns exceed the grid", F);
        e = qs_launch_dependent(gated_act_kernel<bf16, true>, dim3(rows, by), dim3(threads), 0, stream, (bf16*)out, (size_t)ldo,
                                (const bf16*)ab, (size_t)ldi, F, act);
    } else {
        const int by = (F + 255) / 256;
        QS_REQUIRE(by <= 65535, "gated_act: %d columns exceed the grid", F);
        if (dtype == QS_F32)
            e = qs_launch_dependent(gated_act_kernel<float, false>, dim3(rows, by), dim3(256), 0, stream, (float*)out, (size_t)ldo,
                                    (const float*)ab, (size_t)ldi, F, act);
        else if (dtype == QS_BF16)
            e = qs_launch_dependent(gated_act_kernel<bf16, false>, dim3(rows, by), dim3(256), 0, stream, (bf16*)out, (size_t)ldo,
                                    (const bf16*)ab, (size_t)ldi, F, act);
        else return qs_fail(QS_ERR_INVALID_INPUT, "gated_act: unknown dtype %d", dtype);
    }
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "gated_act: %s", cudaGetErrorString(e));
    return qs_check_launch("gated_act");
}

QS_API int qs_clamped_glu(void* out, long long ldo, const void* ab, long long ldi, int dtype, int rows, int F, float limit,
                          float alpha, float shift, cudaStream_t stream) {
    if (rows == 0) return QS_OK;
    QS_REQUIRE(rows > 0 && F > 0 && ldi >= 2 * (long long)F && ldo >= F, "clamped_glu: bad sizes rows=%d F=%d", rows, F);
    typedef __nv_bfloat16 bf16;
    cudaError_t e;
    if (dtype == QS_BF16 && F % 8 == 0 && ldi % 8 == 0 && ldo % 8 == 0 && ((uintptr_t)ab % 16) == 0 && ((uintptr_t)out % 16) == 0) {
        const int threads = F >= 2048 ? 256 : 64;
        const int by = (F / 8 + threads - 1) / threads;
        QS_REQUIRE(by <= 65535, "clamped_glu: %d columns exceed the grid", F);
        e = qs_launch_dependent(clamped_glu_kernel<bf16, true>, dim3(rows, by), dim3(threads), 0, stream, (bf16*)out, (size_t)ldo,
                                (const bf16*)ab, (size_t)ldi, F, limit, alpha, shift);
    } else {
        const int threads = F >= 256 ? 256 : 64;
        const int by = (F + threads - 1) / threads;
        QS_REQUIRE(by <= 65535, "clamped_glu: %d columns exceed the grid", F);
        if (dtype == QS_F32)
            e = qs_launch_dependent(clamped_glu_kernel<float, false>, dim3(rows, by), dim3(threads), 0, stream, (float*)out, (size_t)ldo,
                                    (const float*)ab, (size_t)ldi, F, limit, alpha, shift);
        else if (dtype == QS_BF16)
            e = qs_launch_dependent(clamped_glu_kernel<bf16, false>, dim3(rows, by), dim3(threads), 0, stream, (bf16*)out, (size_t)ldo,
                                    (const bf16*)ab, (size_t)ldi, F, limit, alpha, shift);
        else return qs_fail(QS_ERR_INVALID_INPUT, "clamped_glu: unknown dtype %d", dtype);
    }
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "clamped_glu: %s", cudaGetErrorString(e));
    return qs_check_launch("clamped_glu");
}

QS_API int qs_activate(void* x, long long ld, int dtype, int rows, int n, int act, cudaStream_t stream) {
    if (rows == 0 || n == 0) return QS_OK;
    QS_REQUIRE(rows > 0 && n > 0 && ld >= n && (n + 255) / 256 <= 65535, "activate: bad sizes rows=%d n=%d", rows, n);
    cudaError_t e;
    if (dtype == QS_F32)
        e = qs_launch_dependent(activate_kernel<float>, dim3(rows, (n + 255) / 256), dim3(256), 0, stream, (float*)x, (size_t)ld, n, act);
    else if (dtype == QS_BF16)
        e = qs_launch_dependent(activate_kernel<__nv_bfloat16>, dim3(rows, (n + 255) / 256), dim3(256), 0, stream,
                                (__nv_bfloat16*)x, (size_t)ld, n, act);
    else return qs_fail(QS_ERR_INVALID_INPUT, "activate: unknown dtype %d", dtype);
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "activate: %s", cudaGetErrorString(e));
    return qs_check_launch("activate");
}

QS_API int qs_embedding_hashed(void* out, int out_dtype, const void* table, const void* pair, int table_dtype, float scale,
                               long long buckets, long long mul_prev, long long mul_cur, const int32_t* tokens,
                               const int32_t* tok_slot, const int32_t* tok_pos, const int32_t* last_token, long long ld_last,
                               int T, int D, int V, cudaStream_t stream) {
    if (T == 0) return QS_OK;
    QS_REQUIRE(T > 0 && D > 0 && V > 0, "embedding: bad sizes T=%d D=%d V=%d", T, D, V);
    QS_REQUIRE(!pair || (buckets > 0 && last_token), "embedding: a pair table needs buckets and the sequences' last tokens");
    const int threads = D >= 1024 ? 256 : 128;
#define LAUNCH(TO, TT) embedding_hashed_kernel<TO, TT><<<T, threads, 0, stream>>>((TO*)out, (const TT*)table, scale, \
        (const TT*)pair, buckets, mul_prev, mul_cur, tokens, tok_slot, tok_pos, last_token, (size_t)ld_last, D, V)
    if (out_dtype == QS_F32 && table_dtype == QS_F32) LAUNCH(float, float);
    else if (out_dtype == QS_F32 && table_dtype == QS_BF16) LAUNCH(float, __nv_bfloat16);
    else if (out_dtype == QS_BF16 && table_dtype == QS_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else return qs_fail(QS_ERR_INVALID_INPUT, "embedding: unsupported types out=%d table=%d", out_dtype, table_dtype);
#undef LAUNCH
    return qs_check_launch("embedding_hashed");
}

QS_API int qs_keep_last_rows(void* dst, long long dst_bytes, const void* src, long long src_bytes, int row_bytes,
                             const int32_t* seq_start, const int32_t* seq_slot, int n_seq, cudaStream_t stream) {
    if (n_seq == 0) return QS_OK;
    QS_REQUIRE(n_seq > 0 && row_bytes > 0 && row_bytes % 4 == 0 && dst_bytes % 4 == 0 && src_bytes % 4 == 0 &&
               ((uintptr_t)dst % 4) == 0 && ((uintptr_t)src % 4) == 0, "keep_last_rows: rows must be whole 4-byte words");
    const int words = row_bytes / 4;
    keep_last_rows_kernel<<<n_seq, words >= 256 ? 256 : (words >= 64 ? 64 : 32), 0, stream>>>(
        (uint32_t*)dst, (size_t)dst_bytes / 4, (const uint32_t*)src, (size_t)src_bytes / 4, words, seq_start, seq_slot);
    return qs_check_launch("keep_last_rows");
}
