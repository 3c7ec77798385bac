// Routed experts: the router's choice, and the two ways the chosen experts run.
//
//   moe_route     per token: scores s = sigmoid(z); choice scores s + correction; experts in equal groups of
//                 neighbours, a group's score the sum of its two largest choice scores, only the best `keep` groups
//                 stay (the others count as minus infinity); the `top` largest choice scores win (equal scores: the
//                 lower index); weights s * scale of the winners, not renormalised; optionally sigmoid of one more
//                 logit per token (the gate of a shared expert).  `score_kind` 1: s = softmax(z) over all experts
//                 instead of the sigmoid; `group_kind` 1: a group's score is its largest choice score
//   few tokens    moe_expert_up / moe_expert_down: every (token, chosen expert) pair reads its expert's matrices
//                 through the routing table on the device, so a step can be captured and replayed
//   many tokens   moe_sort orders the pairs by expert; the caller runs one matrix product per expert over its rows
//                 and moe_combine adds each token's weighted results
//
// Router arithmetic, weights and all sums are 32-bit; a token's sum runs over its experts in the order of choice.
#include "common.cuh"

namespace {

constexpr int MAX_EXPERTS = 1024;

// One warp per token.  Lanes compute the scores; lane 0 selects.
__global__ void moe_route_kernel(int32_t* __restrict__ idx, float* __restrict__ wts, float* __restrict__ shared_gate,
                                 const float* __restrict__ z, size_t ldz, const void* __restrict__ corr, int corr_dtype,
                                 int T, int E, int top, int groups, int keep, float scale, int gate_col, int score_kind,
                                 int group_kind) {
    extern __shared__ float sm[];                       // per warp: s [E], choice [E], group score [groups]
    grid_dep_launch();
    grid_dep_wait();
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * warps + warp;
    if (t >= T) return;
    float* s = sm + (size_t)warp * (2 * E + groups);
    float* choice = s + E;
    float* gscore = choice + E;
    const float* zr = z + (size_t)t * ldz;
    float z_max = -INFINITY, inv_sum = 1.0f;
    if (score_kind == 1) {                              // softmax over all experts: the largest logit, then the sum
        for (int e = lane; e < E; e += 32) z_max = fmaxf(z_max, zr[e]);
        for (int off = 16; off > 0; off >>= 1) z_max = fmaxf(z_max, __shfl_xor_sync(0xffffffffu, z_max, off));
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) sum += expf(zr[e] - z_max);
        inv_sum = 1.0f / warp_sum(sum);
    }
    for (int e = lane; e < E; e += 32) {
        s[e] = score_kind == 1 ? expf(zr[e] - z_max) * inv_sum : sigmoid_f32(zr[e]);
        choice[e] = s[e] + (corr ? load_as_f32(corr, corr_dtype, e) : 0.f);
    }
    if (shared_gate && lane == 0 && gate_col >= 0) shared_gate[t] = sigmoid_f32(zr[gate_col]);
    __syncwarp();
    const int per = E / groups;
    if (keep < groups) {
        for (int g = lane; g < groups; g += 32) {
            float a = -INFINITY, b = -INFINITY;          // the two largest
            for (int e = g * per; e < (g + 1) * per; ++e) {
                const float c = choice[e];
                if (c > a) { b = a; a = c; } else if (c > b) b = c;
            }
            gscore[g] = (per > 1 && group_kind == 0) ? a + b : a;
        }
        __syncwarp();
        if (lane == 0) {
            // keep the best `keep` groups: drop the others' experts
            for (int n = 0; n < groups - keep; ++n) {
                int worst = -1;
                for (int g = 0; g < groups; ++g)            // the lowest score; among equals the highest index goes
                    if (gscore[g] != INFINITY && (worst < 0 || gscore[g] <= gscore[worst])) worst = g;
                gscore[worst] = INFINITY;                   // marks a dropped group
                for (int e = worst * per; e < (worst + 1) * per; ++e) choice[e] = -INFINITY;
            }
        }
        __syncwarp();
    }
    if (lane == 0) {
        for (int j = 0; j < top; ++j) {
            int best = -1;
            for (int e = 0; e < E; ++e)
                if (choice[e] != -INFINITY && (best < 0 || choice[e] > choice[best])) best = e;
            if (best < 0) best = 0;                         // fewer live experts than `top`: cannot happen with a sound config
            idx[(size_t)t * top + j] = best;
            wts[(size_t)t * top + j] = s[best] * scale;
            choice[best] = -INFINITY;
        }
    }
}

// sum_k w[k] * x[k] over a warp: lanes take pieces of eight elements (16-byte loads of bfloat16, two of float32)
// where `vec` says that K is a multiple of 8 and the row is aligned, else single elements.
template <typename T>
__device__ __forceinline__ float warp_dot(const T* __restrict__ w, const float* __restrict__ x, int K, int lane, bool vec) {
    float acc = 0.f;
    if (vec) {
        for (int k = lane * 8; k < K; k += 256) {
            float wv[8];
            load8_as_f32(w, sizeof(T) == 4 ? QS_F32 : QS_BF16, k, wv);
            const float4 a = *reinterpret_cast<const float4*>(x + k), b = *reinterpret_cast<const float4*>(x + k + 4);
            acc = fmaf(wv[0], a.x, acc); acc = fmaf(wv[1], a.y, acc); acc = fmaf(wv[2], a.z, acc); acc = fmaf(wv[3], a.w, acc);
            acc = fmaf(wv[4], b.x, acc); acc = fmaf(wv[5], b.y, acc); acc = fmaf(wv[6], b.z, acc); acc = fmaf(wv[7], b.w, acc);
        }
    } else {
        for (int k = lane; k < K; k += 32) acc = fmaf(to_f32(w[k]), x[k], acc);
    }
    return warp_sum(acc);
}

// hidden[pair, f] = act(W_up[e][f, :] . h[token, :]) for pair = token * top + j, e = idx[pair]: a block stages the
// token's row in shared memory as 32-bit floats, a warp takes one hidden unit at a time.
template <typename T>
__global__ void moe_expert_up_kernel(T* __restrict__ hidden, size_t ldh, const T* __restrict__ x, size_t ldx,
                                     const T* __restrict__ w_up, const int32_t* __restrict__ idx,
                                     const int32_t* __restrict__ tok_slot, int top, int D, int F, int rows_per_block, int act,
                                     int vec) {
    extern __shared__ __align__(16) float xs[];
    grid_dep_launch();
    grid_dep_wait();
    const int pair = blockIdx.x, t = pair / top;
    const int f0 = blockIdx.y * rows_per_block;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    if (tok_slot[t] < 0) {
        for (int f = f0 + threadIdx.x; f < min(F, f0 + rows_per_block); f += blockDim.x) hidden[(size_t)pair * ldh + f] = from_f32<T>(0.f);
        return;
    }
    for (int i = threadIdx.x; i < D; i += blockDim.x) xs[i] = to_f32(x[(size_t)t * ldx + i]);
    __syncthreads();
    const T* w = w_up + (size_t)idx[pair] * F * D;
    for (int f = f0 + warp; f < min(F, f0 + rows_per_block); f += warps) {
        const float acc = warp_dot(w + (size_t)f * D, xs, D, lane, vec != 0);
        if (lane == 0) hidden[(size_t)pair * ldh + f] = from_f32<T>(apply_activation_wide(acc, act));
    }
}

// out[t, d] = sum_j wts[t, j] * (W_down[idx[t, j]][d, :] . hidden[t * top + j, :])  (+ add[t, d] * add_scale[t]),
// 32-bit.  A block stages the token's `top` hidden rows; a warp takes one output element at a time.
template <typename T>
__global__ void moe_expert_down_kernel(float* __restrict__ out, size_t ldo, const T* __restrict__ hidden, size_t ldh,
                                       const T* __restrict__ w_down, const int32_t* __restrict__ idx,
                                       const float* __restrict__ wts, const int32_t* __restrict__ tok_slot,
                                       const void* __restrict__ add, int add_dtype, size_t ldadd,
                                       const float* __restrict__ add_scale, int top, int D, int F, int rows_per_block,
                                       int vec) {
    extern __shared__ __align__(16) float hs[];         // [top][F]
    grid_dep_launch();
    grid_dep_wait();
    const int t = blockIdx.x;
    const int d0 = blockIdx.y * rows_per_block;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    if (tok_slot[t] < 0) {
        for (int d = d0 + threadIdx.x; d < min(D, d0 + rows_per_block); d += blockDim.x) out[(size_t)t * ldo + d] = 0.f;
        return;
    }
    for (int i = threadIdx.x; i < top * F; i += blockDim.x) {
        const int j = i / F;
        hs[i] = to_f32(hidden[((size_t)t * top + j) * ldh + (i - j * F)]);
    }
    __syncthreads();
    for (int d = d0 + warp; d < min(D, d0 + rows_per_block); d += warps) {
        float total = 0.f;
        for (int j = 0; j < top; ++j) {
            const T* wr = w_down + ((size_t)idx[(size_t)t * top + j] * D + d) * F;
            total = fmaf(wts[(size_t)t * top + j], warp_dot(wr, hs + j * F, F, lane, vec != 0), total);
        }
        if (lane == 0) {
            if (add) total = fmaf(load_as_f32(add, add_dtype, (size_t)t * ldadd + d), add_scale ? add_scale[t] : 1.0f, total);
            out[(size_t)t * ldo + d] = total;
        }
    }
}

// The (token, choice) pairs ordered by expert, by one block: offsets[e] .. offsets[e + 1] are expert e's places,
// place_token[p] the token whose row goes there, pair_place[pair] the place of a pair.  Pairs of padding rows
// (slot < 0) are counted for the expert they name: their rows are zeros and nobody reads their results.
__global__ void moe_sort_kernel(int32_t* __restrict__ offsets, int32_t* __restrict__ place_token,
                                int32_t* __restrict__ pair_place, const int32_t* __restrict__ idx, int n_pairs, int top, int E) {
    __shared__ int count[MAX_EXPERTS + 1];
    for (int e = threadIdx.x; e <= E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) atomicAdd(&count[idx[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) { const int c = count[e]; offsets[e] = run; count[e] = run; run += c; }
        offsets[E] = run;
    }
    __syncthreads();
    // a pair's place inside its expert's range is whatever the counter gives it: a row's products do not depend
    // on where the row lies, so the order is free
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int place = atomicAdd(&count[idx[p]], 1);
        place_token[place] = p / top;
        pair_place[p] = place;
    }
}

// out[t, :] = sum_j wts[t, j] * y[pair_place[t * top + j], :]  (+ add[t, :] * add_scale[t]), in 32-bit.
template <typename TY>
__global__ void moe_combine_kernel(float* __restrict__ out, size_t ldo, const TY* __restrict__ y, size_t ldy,
                                   const int32_t* __restrict__ pair_place, const float* __restrict__ wts,
                                   const int32_t* __restrict__ tok_slot, const void* __restrict__ add, int add_dtype,
                                   size_t ldadd, const float* __restrict__ add_scale, int top, int D) {
    grid_dep_launch();
    grid_dep_wait();
    const size_t t = blockIdx.x;
    const bool live = tok_slot[t] >= 0;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float total = 0.f;
        if (live) {
            for (int j = 0; j < top; ++j)
                total = fmaf(wts[t * top + j], to_f32(y[(size_t)pair_place[t * top + j] * ldy + d]), total);
            if (add) total = fmaf(load_as_f32(add, add_dtype, t * ldadd + d), add_scale ? add_scale[t] : 1.0f, total);
        }
        out[t * ldo + d] = total;
    }
}

}  // namespace

QS_API int qs_moe_route(int32_t* idx, float* wts, float* shared_gate, const float* z, long long ldz, const void* corr,
                        int corr_dtype, int T, int E, int top, int groups, int keep, float scale, int gate_col,
                        int score_kind, int group_kind, cudaStream_t stream) {
    if (T == 0) return QS_OK;
    QS_REQUIRE(T > 0 && E > 0 && E <= MAX_EXPERTS && top > 0 && top <= E, "moe_route: bad sizes T=%d E=%d top=%d", T, E, top);
    QS_REQUIRE(groups > 0 && E % groups == 0 && keep > 0 && keep <= groups, "moe_route: %d experts in %d groups, %d kept", E, groups, keep);
    QS_REQUIRE(keep * (E / groups) >= top, "moe_route: %d kept groups of %d experts cannot give %d choices", keep, E / groups, top);
    const int warps = 4;
    const size_t smem = (size_t)warps * (2 * E + groups) * sizeof(float);
    cudaError_t e = qs_launch_dependent(moe_route_kernel, dim3((T + warps - 1) / warps), dim3(warps * 32), smem, stream, idx, wts,
                                        shared_gate, z, (size_t)ldz, corr, corr_dtype, T, E, top, groups, keep, scale, gate_col, score_kind,
                                        group_kind);
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "moe_route: %s", cudaGetErrorString(e));
    return qs_check_launch("moe_route");
}

QS_API int qs_moe_expert_up(void* hidden, long long ldh, const void* x, long long ldx, const void* w_up, int dtype,
                            const int32_t* idx, const int32_t* tok_slot, int T, int top, int D, int F, int act,
                            cudaStream_t stream) {
    if (T == 0) return QS_OK;
    QS_REQUIRE(T > 0 && top > 0 && D > 0 && F > 0, "moe_expert_up: bad sizes");
    QS_REQUIRE((size_t)D * sizeof(float) <= 200 * 1024, "moe_expert_up: width %d does not fit shared memory", D);
    const int rows_per_block = 32;
    const size_t smem = (size_t)D * sizeof(float);
    const int vec = D % 8 == 0 && ((uintptr_t)w_up % 16) == 0;
    dim3 grid(T * top, (F + rows_per_block - 1) / rows_per_block);
    cudaError_t e = cudaSuccess;
#define GO(TT) do { if (smem > 48 * 1024) e = cudaFuncSetAttribute(moe_expert_up_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    if (e == cudaSuccess) e = qs_launch_dependent(moe_expert_up_kernel<TT>, grid, dim3(256), smem, stream, (TT*)hidden, (size_t)ldh, (const TT*)x, \
        (size_t)ldx, (const TT*)w_up, idx, tok_slot, top, D, F, rows_per_block, act, vec); } while (0)
    if (dtype == QS_F32) GO(float);
    else if (dtype == QS_BF16) GO(__nv_bfloat16);
    else return qs_fail(QS_ERR_INVALID_INPUT, "moe_expert_up: unknown dtype %d", dtype);
#undef GO
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "moe_expert_up: %s", cudaGetErrorString(e));
    return qs_check_launch("moe_expert_up");
}

QS_API int qs_moe_expert_down(float* out, long long ldo, const void* hidden, long long ldh, const void* w_down, int dtype,
                              const int32_t* idx, const float* wts, const int32_t* tok_slot, const void* add, int add_dtype,
                              long long ldadd, const float* add_scale, int T, int top, int D, int F, cudaStream_t stream) {
    if (T == 0) return QS_OK;
    QS_REQUIRE(T > 0 && top > 0 && D > 0 && F > 0, "moe_expert_down: bad sizes");
    const size_t smem = (size_t)top * F * sizeof(float);
    QS_REQUIRE(smem <= 200 * 1024, "moe_expert_down: %d x %d hidden values do not fit shared memory", top, F);
    const int rows_per_block = 32;
    const int vec = F % 8 == 0 && ((uintptr_t)w_down % 16) == 0;
    dim3 grid(T, (D + rows_per_block - 1) / rows_per_block);
    cudaError_t e = cudaSuccess;
#define GO(TT) do { if (smem > 48 * 1024) e = cudaFuncSetAttribute(moe_expert_down_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    if (e == cudaSuccess) e = qs_launch_dependent(moe_expert_down_kernel<TT>, grid, dim3(256), smem, stream, out, (size_t)ldo, (const TT*)hidden, \
        (size_t)ldh, (const TT*)w_down, idx, wts, tok_slot, add, add_dtype, (size_t)ldadd, add_scale, top, D, F, rows_per_block, vec); } while (0)
    if (dtype == QS_F32) GO(float);
    else if (dtype == QS_BF16) GO(__nv_bfloat16);
    else return qs_fail(QS_ERR_INVALID_INPUT, "moe_expert_down: unknown dtype %d", dtype);
#undef GO
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "moe_expert_down: %s", cudaGetErrorString(e));
    return qs_check_launch("moe_expert_down");
}

QS_API int qs_moe_sort(int32_t* offsets, int32_t* place_token, int32_t* pair_place, const int32_t* idx, int n_pairs,
                       int top, int E, cudaStream_t stream) {
    QS_REQUIRE(n_pairs > 0 && top > 0 && E > 0 && E <= MAX_EXPERTS, "moe_sort: bad sizes");
    moe_sort_kernel<<<1, 1024, 0, stream>>>(offsets, place_token, pair_place, idx, n_pairs, top, E);
    return qs_check_launch("moe_sort");
}

QS_API int qs_moe_combine(float* out, long long ldo, const void* y, int y_dtype, long long ldy, const int32_t* pair_place,
                          const float* wts, const int32_t* tok_slot, const void* add, int add_dtype, long long ldadd,
                          const float* add_scale, int T, int top, int D, cudaStream_t stream) {
    if (T == 0) return QS_OK;
    QS_REQUIRE(T > 0 && top > 0 && D > 0, "moe_combine: bad sizes");
    const int threads = D >= 1024 ? 256 : 128;
    cudaError_t e;
#define GO(TY) e = qs_launch_dependent(moe_combine_kernel<TY>, dim3(T), dim3(threads), 0, stream, out, (size_t)ldo, (const TY*)y, \
        (size_t)ldy, pair_place, wts, tok_slot, add, add_dtype, (size_t)ldadd, add_scale, top, D)
    if (y_dtype == QS_F32) GO(float);
    else if (y_dtype == QS_BF16) GO(__nv_bfloat16);
    else return qs_fail(QS_ERR_INVALID_INPUT, "moe_combine: unknown dtype %d", y_dtype);
#undef GO
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "moe_combine: %s", cudaGetErrorString(e));
    return qs_check_launch("moe_combine");
}

// The matrix products of the library (csrc/gemm_tc.cu, csrc/linear_simt.cu).
extern "C" int qs_gemm_tc(void* C, int c_dtype, const void* A, const void* W, const void* bias, int bias_dtype, int act,
                          const void* res1, const void* res2, int M, int N, int K, long long lda, long long ldw,
                          long long ldc, long long ldr, float* ws, long long ws_floats, int32_t* counters, int n_counters,
                          int32_t* status, int smem_kb, cudaStream_t stream);
extern "C" int qs_linear_simt(void* C, int c_dtype, const void* A, int a_dtype, const void* W, int w_dtype,
                              const void* bias, int bias_dtype, int act, const void* res1, const void* res2,
                              int M, int N, int K, long long lda, long long ldc, long long ldr, cudaStream_t stream);

// One product per expert over its rows, all launched by this one call: C[rows of e] = A[rows of e] W[e]^T with
// W [E][N][K] and the experts' row ranges `offsets` (E + 1 entries, on the HOST).  `use_tc`: the tensor-core product
// (bfloat16 operands that it takes) with its scratch `ws`, `counters`, `status`; else the CUDA-core product.
//
// An expert's product is small (a thousand rows fill a sixth of the SMs with tiles), so the experts are dealt to
// EXPERT_STREAMS streams of the library's own that fork from `stream` and join it again before the call returns; each
// stream has its own share of the scratch.  While `stream` is being captured everything stays on it, in order.
namespace {
constexpr int EXPERT_STREAMS = 8, MAX_DEVICES = 16;
struct ExpertStreams { cudaStream_t side[EXPERT_STREAMS]; cudaEvent_t fork, join[EXPERT_STREAMS]; bool ready; };
ExpertStreams g_expert_streams[MAX_DEVICES];

ExpertStreams* expert_streams() {
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= MAX_DEVICES) return nullptr;
    ExpertStreams& p = g_expert_streams[device];
    if (!p.ready) {
        if (cudaEventCreateWithFlags(&p.fork, cudaEventDisableTiming) != cudaSuccess) return nullptr;
        for (int i = 0; i < EXPERT_STREAMS; ++i)
            if (cudaStreamCreateWithFlags(&p.side[i], cudaStreamNonBlocking) != cudaSuccess ||
                cudaEventCreateWithFlags(&p.join[i], cudaEventDisableTiming) != cudaSuccess) return nullptr;
        p.ready = true;
    }
    return &p;
}
}  // namespace

QS_API int qs_expert_products(void* C, int c_dtype, long long ldc, const void* A, int a_dtype, long long lda, const void* W,
                              int w_dtype, const int32_t* offsets, int E, int N, int K, int use_tc, float* ws,
                              long long ws_floats, int32_t* counters, int n_counters, int32_t* status, cudaStream_t stream) {
    QS_REQUIRE(E > 0 && N > 0 && K > 0 && offsets, "expert_products: bad sizes");
    const size_t a_size = a_dtype == QS_F32 ? 4 : 2, c_size = c_dtype == QS_F32 ? 4 : 2, w_size = w_dtype == QS_F32 ? 4 : 2;
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    ExpertStreams* pool = nullptr;
    if (E > 1 && cudaStreamIsCapturing(stream, &capturing) == cudaSuccess && capturing == cudaStreamCaptureStatusNone)
        pool = expert_streams();
    const int lanes = pool ? EXPERT_STREAMS : 1;
    const long long ws_share = ws_floats / lanes / 4 * 4;
    const int counter_share = n_counters / lanes;
    if (pool) {
        if (cudaEventRecord(pool->fork, stream) != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "expert_products: cannot fork");
        for (int i = 0; i < lanes; ++i) cudaStreamWaitEvent(pool->side[i], pool->fork, 0);
    }
    int rc = QS_OK;
    for (int e = 0; e < E && rc == QS_OK; ++e) {
        const int lo = offsets[e], M = offsets[e + 1] - lo;
        if (M <= 0) continue;
        const int lane = e % lanes;
        cudaStream_t st = pool ? pool->side[lane] : stream;
        char* c = (char*)C + (size_t)lo * ldc * c_size;
        const char* a = (const char*)A + (size_t)lo * lda * a_size;
        const char* w = (const char*)W + (size_t)e * N * K * w_size;
        rc = use_tc ? qs_gemm_tc(c, c_dtype, a, w, nullptr, 0, QS_ACT_NONE, nullptr, nullptr, M, N, K, lda, K, ldc, N,
                                 ws + (size_t)lane * ws_share, ws_share, counters + (size_t)lane * counter_share, counter_share,
                                 status, 0, st)
                    : qs_linear_simt(c, c_dtype, a, a_dtype, w, w_dtype, nullptr, 0, QS_ACT_NONE, nullptr, nullptr, M, N, K, lda,
                                     ldc, N, st);
    }
    if (pool)                                           // also after a failed launch: `stream` must not run ahead of the others
        for (int i = 0; i < lanes; ++i) {
            cudaEventRecord(pool->join[i], pool->side[i]);
            cudaStreamWaitEvent(stream, pool->join[i], 0);
        }
    return rc;
}

// One product per head over the same rows, dealt to the same streams: C[:, head h] = A[:, head h] W[h]^T with W [H][N][K],
// head h's K inputs at A + h * head_a and its N results at C + h * head_c (elements), rows `lda` and `ldc` apart.
QS_API int qs_head_products(void* C, int c_dtype, long long ldc, long long head_c, const void* A, int a_dtype, long long lda,
                            long long head_a, const void* W, int w_dtype, int M, int H, int N, int K, int use_tc, float* ws,
                            long long ws_floats, int32_t* counters, int n_counters, int32_t* status, cudaStream_t stream) {
    QS_REQUIRE(M > 0 && H > 0 && N > 0 && K > 0, "head_products: bad sizes");
    const size_t a_size = a_dtype == QS_F32 ? 4 : 2, c_size = c_dtype == QS_F32 ? 4 : 2, w_size = w_dtype == QS_F32 ? 4 : 2;
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    ExpertStreams* pool = nullptr;
    if (H > 1 && cudaStreamIsCapturing(stream, &capturing) == cudaSuccess && capturing == cudaStreamCaptureStatusNone)
        pool = expert_streams();
    const int lanes = pool ? EXPERT_STREAMS : 1;
    const long long ws_share = ws_floats / lanes / 4 * 4;
    const int counter_share = n_counters / lanes;
    if (pool) {
        if (cudaEventRecord(pool->fork, stream) != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "head_products: cannot fork");
        for (int i = 0; i < lanes; ++i) cudaStreamWaitEvent(pool->side[i], pool->fork, 0);
    }
    int rc = QS_OK;
    for (int h = 0; h < H && rc == QS_OK; ++h) {
        const int lane = h % lanes;
        cudaStream_t st = pool ? pool->side[lane] : stream;
        char* c = (char*)C + (size_t)h * head_c * c_size;
        const char* a = (const char*)A + (size_t)h * head_a * a_size;
        const char* w = (const char*)W + (size_t)h * N * K * w_size;
        rc = use_tc ? qs_gemm_tc(c, c_dtype, a, w, nullptr, 0, QS_ACT_NONE, nullptr, nullptr, M, N, K, lda, K, ldc, N,
                                 ws + (size_t)lane * ws_share, ws_share, counters + (size_t)lane * counter_share, counter_share,
                                 status, 0, st)
                    : qs_linear_simt(c, c_dtype, a, a_dtype, w, w_dtype, nullptr, 0, QS_ACT_NONE, nullptr, nullptr, M, N, K, lda,
                                     ldc, N, st);
    }
    if (pool)
        for (int i = 0; i < lanes; ++i) {
            cudaEventRecord(pool->join[i], pool->side[i]);
            cudaStreamWaitEvent(stream, pool->join[i], 0);
        }
    return rc;
}
