// Mixers that carry a matrix of state per head from token to token, and the token shift in front of one of them.
//
//   linear attention with a fixed decay per head ("lightning"):
//       S_t = decay_h S_{t-1} + k_t v_t^T,   o_t = S_t^T q_t                   q, k [dk], v, o [dv], S [dk, dv]
//   time mixing with a decay per token and key channel and a bonus for the current token ("wkv"):
//       o_t = (S_{t-1} + diag(u) k_t v_t^T)^T r_t,   S_t = diag(w_t) S_{t-1} + k_t v_t^T,   w_t = exp(-exp(d_t))
//   matrix memory with a decay and an input weight per token and head ("gated"; the mLSTM's recurrence once its
//   gates are turned into the factors a_t, b_t by `mlstm_gates_kernel`):
//       S_t = a_t S_{t-1} + b_t k_t v_t^T,   o_t = S_t^T (q_t * q_scale);   the last column of S has v = 1 and so
//       carries the normaliser n_t = a_t n_{t-1} + b_t k_t, whose product with q arrives as the last element of o
//   delta rule with a decay per token and key channel and a step size per token and head ("delta"):
//       S' = diag(g_t) S_{t-1},   u_t = beta_t (v_t - S'^T k_t),   S_t = S' + k_t u_t^T,   o_t = S_t^T q_t
//       (q, k, v arrive ready: activated, normed, scaled; several heads may share one head of q and k).  A column of S
//       does not meet the others, so the threads of a column pair take S'^T k, S'^T q and k.q in one round of
//       shuffles, and o_t = S'^T q + u_t (k.q).  In order only (PHASE 0).
//   gated linear attention with a decay per token and key channel ("gla"):
//       S_t = diag(w_t) S_{t-1} + k_t v_t^T,   o_t = S_t^T (q_t * q_scale),   w_t = sigmoid(z_t)^decay_scale
//       (the decay acts before the token's own output, where "wkv" applies it after)
//
// The state lives in 32-bit, per slot as [heads][dv][dk] (a column of S is contiguous), starts at zero and is
// read at the start of a step and written back at its end; everything between the projections and the output is
// 32-bit arithmetic.  One kernel serves prompts and single tokens: a block owns some columns of one head of one
// sequence and walks the sequence's tokens of this step in order.  A thread owns RK key rows of two neighbouring
// columns; the KS threads of a pair of columns are neighbours in a warp and add their parts of o by shuffles, in a
// fixed order, so a token's result does not depend on the batch or on how the prompt was cut.
#include "common.cuh"

namespace {

constexpr int RK = 16;              // key rows per thread and column
constexpr int CPT = 2;              // columns per thread: a token's q and k are read from shared memory once for both
constexpr int TILE = 16;            // tokens staged in shared memory at a time

// Which rows a thread owns: groups of four consecutive rows, dealt to the KS threads of a column in turn, so that
// the threads' 16-byte accesses to a column of the state and to a token's q and k lie side by side.
__device__ __forceinline__ float log_sigmoid_f32(float z) { return z >= 0.f ? -log1pf(expf(-z)) : z - log1pf(expf(z)); }

__device__ __forceinline__ int row_of(int ks, int ks_log2, int r) { return 4 * (ks + ((r >> 2) << ks_log2)) + (r & 3); }

// PHASE 0: a sequence's tokens in order from the state its slot holds, which is written back at the end.
// A long prompt is cut into chunks that run side by side, in three steps whose sums are 32-bit throughout:
// PHASE 1: every chunk by itself from a zero state (its own part of every o, and the state it adds); then
//          `chunk_prefix_kernel` walks each sequence's chunks, replacing each chunk's added state by the state
//          the chunk starts from and leaving the sequence's last state in its slot;
// PHASE 3: every chunk adds to its tokens' o what the state it started from contributes, decayed up to each token.
// For phases 1 and 3 a "sequence" of the kernel is a chunk and its "slot" the chunk's place in the scratch.
template <typename TI, int MODE, int PHASE>
__global__ void __launch_bounds__(256, 2)
state_scan_kernel(float* __restrict__ o, size_t ldo,
                  const TI* __restrict__ q, size_t ldq, const TI* __restrict__ k, size_t ldk,
                  const TI* __restrict__ v, size_t ldv, const float* __restrict__ dlog, size_t ldd,
                  const float* __restrict__ head_decay, const void* __restrict__ bonus, int bonus_dtype,
                  float* __restrict__ state, size_t slot_stride,
                  const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_slot, int n_seq, int T_rows,
                  int H, int dk, int dv, int ks_log2, int cols, int in_act, int vec,
                  const float* __restrict__ ga, const float* __restrict__ gb, size_t ldg, float q_scale, int qk_group,
                  float decay_scale) {
    constexpr bool WKV = MODE == 1, GATED = MODE == 2, DELTA = MODE == 3, GLA = MODE == 4;
    extern __shared__ float smem[];
    const int KS = 1 << ks_log2, dkp = KS * RK;
    float* sq = smem;                                   // [TILE][dkp]
    float* sk = sq + TILE * dkp;                        // [TILE][dkp]
    float* sw = sk + TILE * dkp;                        // [TILE][dkp]   (WKV only)
    float* sv = sw + (WKV || DELTA || GLA ? TILE * dkp : 0);   // [TILE][cols]
    float* carry = sv + TILE * cols;                    // [dkp]         (PHASE 3: the decay from the chunk's start on)
    float* sa = carry + dkp;                            // [TILE]        (GATED: the tokens' decays)
    const int dvv = GATED ? dv - 1 : dv;                // columns that v holds per head: the gated form adds one of ones
    grid_dep_launch();
    grid_dep_wait();
    const int s = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * cols;
    const int hq = DELTA ? h / qk_group : h;            // the head of q and k that this head reads
    const int n_cols = min(cols, dv - col0);
    const int tid = threadIdx.x;
    // rows of the packed batch beyond the last sequence belong to nobody: give them a defined value
    if (PHASE != 3 && s == 0 && (!DELTA || o)) {
        for (int t = seq_start[n_seq]; t < T_rows; ++t)
            for (int c = tid; c < n_cols; c += blockDim.x) o[(size_t)t * ldo + h * dv + col0 + c] = 0.f;
    }
    const int slot = seq_slot[s];
    const int t0 = seq_start[s], t1 = seq_start[s + 1];
    if (slot < 0) {
        if (PHASE != 3 && (!DELTA || o))
            for (int t = t0; t < t1; ++t)
                for (int c = tid; c < n_cols; c += blockDim.x) o[(size_t)t * ldo + h * dv + col0 + c] = 0.f;
        return;
    }
    if (t1 <= t0) return;
    const int pair = tid >> ks_log2, ks = tid & (KS - 1);
    const bool own0 = CPT * pair < n_cols, own1 = CPT * pair + 1 < n_cols;
    float* scol0 = state + (size_t)slot * slot_stride + ((size_t)h * dv + col0 + (own0 ? CPT * pair : 0)) * dk;
    float* scol1 = state + (size_t)slot * slot_stride + ((size_t)h * dv + col0 + (own1 ? CPT * pair + 1 : 0)) * dk;

    float S0[RK], S1[RK], u[RK];
#pragma unroll
    for (int r4 = 0; r4 < RK / 4; ++r4) {
        const int i = row_of(ks, ks_log2, 4 * r4);
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f), y = x;
        if (PHASE != 1) {
            if (vec) {
                if (own0 && i < dk) x = *reinterpret_cast<const float4*>(scol0 + i);
                if (own1 && i < dk) y = *reinterpret_cast<const float4*>(scol1 + i);
            } else {
                if (own0) { if (i < dk) x.x = scol0[i]; if (i + 1 < dk) x.y = scol0[i + 1]; if (i + 2 < dk) x.z = scol0[i + 2]; if (i + 3 < dk) x.w = scol0[i + 3]; }
                if (own1) { if (i < dk) y.x = scol1[i]; if (i + 1 < dk) y.y = scol1[i + 1]; if (i + 2 < dk) y.z = scol1[i + 2]; if (i + 3 < dk) y.w = scol1[i + 3]; }
            }
        }
        S0[4 * r4] = x.x; S0[4 * r4 + 1] = x.y; S0[4 * r4 + 2] = x.z; S0[4 * r4 + 3] = x.w;
        S1[4 * r4] = y.x; S1[4 * r4 + 1] = y.y; S1[4 * r4 + 2] = y.z; S1[4 * r4 + 3] = y.w;
#pragma unroll
        for (int j = 0; j < 4; ++j)
            u[4 * r4 + j] = (WKV && PHASE != 3 && i + j < dk) ? load_as_f32(bonus, bonus_dtype, (size_t)h * dk + i + j) : 0.f;
    }
    const float decay = (WKV || GATED || GLA) ? 0.f : head_decay[h];
    if (PHASE == 3)
        for (int i = tid; i < dkp; i += blockDim.x) carry[i] = 1.0f;

    for (int base = t0; base < t1; base += TILE) {
        const int nt = min(TILE, t1 - base);
        __syncthreads();
        // a thread stages one key row of the tile's tokens, in order: in PHASE 3 the row's decay since the chunk's
        // start runs along and q arrives multiplied by it
        for (int i = tid; i < dkp; i += blockDim.x) {
            // all of the tile's loads first, so that they are in flight together
            TI qraw[TILE], kraw[TILE];
            float draw[TILE];                           // GATED: b_t (phases 0, 1) or a_t (phase 3)
#pragma unroll
            for (int tt = 0; tt < TILE; ++tt) {
                if (tt < nt && i < dk) {
                    const size_t row = (size_t)(base + tt);
                    qraw[tt] = q[row * ldq + hq * dk + i];
                    if (PHASE != 3) kraw[tt] = k[row * ldk + hq * dk + i];
                    if (WKV || DELTA || GLA) draw[tt] = dlog[row * ldd + h * dk + i];
                    if (GATED) draw[tt] = (PHASE == 3 ? ga : gb)[row * ldg + h];
                }
            }
            float run = PHASE == 3 ? carry[i] : 1.0f;
#pragma unroll
            for (int tt = 0; tt < TILE; ++tt) {
                if (tt < nt) {
                    float qv = 0.f, kv = 0.f, wv = 0.f;
                    if (i < dk) {
                        qv = apply_activation(to_f32(qraw[tt]), in_act);
                        if (PHASE != 3) kv = apply_activation(to_f32(kraw[tt]), in_act);
                        if (WKV) wv = expf(-expf(draw[tt]));
                        if (DELTA) wv = draw[tt];
                        if (GLA) wv = expf(log_sigmoid_f32(draw[tt]) * decay_scale);
                        if (!WKV && !DELTA) qv *= q_scale;      // a constant factor on q (or, the sums being bilinear, on k)
                        if (GATED && PHASE != 3) kv *= draw[tt];
                    }
                    if (PHASE == 3) {
                        if (WKV) { qv *= run; run *= wv; }
                        else if (GLA) { run *= wv; qv *= run; }
                        else if (GATED) { run *= (i < dk ? draw[tt] : 0.f); qv *= run; }
                        else { run *= decay; qv *= run; }
                    } else {
                        sk[tt * dkp + i] = kv;
                        if (WKV || DELTA || GLA) sw[tt * dkp + i] = wv;
                    }
                    sq[tt * dkp + i] = qv;
                }
            }
            if (PHASE == 3) carry[i] = run;
        }
        if (PHASE != 3) {
            for (int e = tid; e < nt * cols; e += blockDim.x) {
                const int tt = e / cols, c = e - tt * cols;
                sv[e] = (c >= n_cols || (DELTA && !v)) ? 0.f : (GATED && col0 + c == dvv) ? 1.0f
                        : apply_activation(to_f32(v[(size_t)(base + tt) * ldv + h * dvv + col0 + c]), in_act);
            }
            if (GATED && tid < nt) sa[tid] = ga[(size_t)(base + tid) * ldg + h];
            if (DELTA && tid < nt) sa[tid] = gb[(size_t)(base + tid) * ldg + h];
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float v0 = (PHASE == 3 || !own0) ? 0.f : sv[tt * cols + CPT * pair];
            const float v1 = (PHASE == 3 || !own1) ? 0.f : sv[tt * cols + CPT * pair + 1];
            const float4* q4 = reinterpret_cast<const float4*>(sq + tt * dkp) + ks;
            const float4* k4 = reinterpret_cast<const float4*>(sk + tt * dkp) + ks;
            const float4* w4 = reinterpret_cast<const float4*>(sw + tt * dkp) + ks;
            float acc0 = 0.f, acc1 = 0.f;
            if (DELTA) {
                float a0 = 0.f, a1 = 0.f, kq = 0.f;
#pragma unroll
                for (int r4 = 0; r4 < RK / 4; ++r4) {
                    const float4 qq = q4[r4 << ks_log2], kk = k4[r4 << ks_log2], ww = w4[r4 << ks_log2];
                    const float qa[4] = {qq.x, qq.y, qq.z, qq.w}, ka[4] = {kk.x, kk.y, kk.z, kk.w}, wa[4] = {ww.x, ww.y, ww.z, ww.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int r = r4 * 4 + j;
                        S0[r] *= wa[j];
                        S1[r] *= wa[j];
                        a0 = fmaf(ka[j], S0[r], a0);
                        a1 = fmaf(ka[j], S1[r], a1);
                        acc0 = fmaf(qa[j], S0[r], acc0);
                        acc1 = fmaf(qa[j], S1[r], acc1);
                        kq = fmaf(ka[j], qa[j], kq);
                    }
                }
                for (int off = KS >> 1; off > 0; off >>= 1) {
                    a0 += __shfl_xor_sync(0xffffffffu, a0, off);
                    a1 += __shfl_xor_sync(0xffffffffu, a1, off);
                    acc0 += __shfl_xor_sync(0xffffffffu, acc0, off);
                    acc1 += __shfl_xor_sync(0xffffffffu, acc1, off);
                    kq += __shfl_xor_sync(0xffffffffu, kq, off);
                }
                const float u0 = sa[tt] * (v0 - a0), u1 = sa[tt] * (v1 - a1);
#pragma unroll
                for (int r4 = 0; r4 < RK / 4; ++r4) {
                    const float4 kk = k4[r4 << ks_log2];
                    const float ka[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        S0[r4 * 4 + j] = fmaf(ka[j], u0, S0[r4 * 4 + j]);
                        S1[r4 * 4 + j] = fmaf(ka[j], u1, S1[r4 * 4 + j]);
                    }
                }
                acc0 = fmaf(u0, kq, acc0);
                acc1 = fmaf(u1, kq, acc1);
            } else {
#pragma unroll
            for (int r4 = 0; r4 < RK / 4; ++r4) {
                const float4 qq = q4[r4 << ks_log2];
                const float qa[4] = {qq.x, qq.y, qq.z, qq.w};
                if (PHASE == 3) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        acc0 = fmaf(qa[j], S0[r4 * 4 + j], acc0);
                        acc1 = fmaf(qa[j], S1[r4 * 4 + j], acc1);
                    }
                } else {
                    const float4 kk = k4[r4 << ks_log2];
                    const float ka[4] = {kk.x, kk.y, kk.z, kk.w};
                    float wa[4] = {0.f, 0.f, 0.f, 0.f};
                    if (WKV || GLA) { const float4 ww = w4[r4 << ks_log2]; wa[0] = ww.x; wa[1] = ww.y; wa[2] = ww.z; wa[3] = ww.w; }
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int r = r4 * 4 + j;
                        const float kv0 = ka[j] * v0, kv1 = ka[j] * v1;
                        if (WKV) {
                            acc0 = fmaf(qa[j], fmaf(u[r], kv0, S0[r]), acc0);
                            acc1 = fmaf(qa[j], fmaf(u[r], kv1, S1[r]), acc1);
                            S0[r] = fmaf(wa[j], S0[r], kv0);
                            S1[r] = fmaf(wa[j], S1[r], kv1);
                        } else if (GLA) {
                            S0[r] = fmaf(wa[j], S0[r], kv0);
                            S1[r] = fmaf(wa[j], S1[r], kv1);
                            acc0 = fmaf(qa[j], S0[r], acc0);
                            acc1 = fmaf(qa[j], S1[r], acc1);
                        } else {
                            const float dec = GATED ? sa[tt] : decay;
                            S0[r] = fmaf(dec, S0[r], kv0);
                            S1[r] = fmaf(dec, S1[r], kv1);
                            acc0 = fmaf(qa[j], S0[r], acc0);
                            acc1 = fmaf(qa[j], S1[r], acc1);
                        }
                    }
                }
            }
            for (int off = KS >> 1; off > 0; off >>= 1) {
                acc0 += __shfl_xor_sync(0xffffffffu, acc0, off);
                acc1 += __shfl_xor_sync(0xffffffffu, acc1, off);
            }
            }
            if (ks == 0 && (!DELTA || o)) {
                // PHASE 3 adds to what PHASE 1 wrote: this thread is the element's only writer in this kernel, and a
                // reduction that returns nothing does not make the loop wait for the old value
                float* dst = o + (size_t)(base + tt) * ldo + h * dv + col0 + CPT * pair;
                if (own0) { if (PHASE == 3) atomicAdd(dst, acc0); else dst[0] = acc0; }
                if (own1) { if (PHASE == 3) atomicAdd(dst + 1, acc1); else dst[1] = acc1; }
            }
        }
    }
    if (PHASE != 3) {
#pragma unroll
        for (int r4 = 0; r4 < RK / 4; ++r4) {
            const int i = row_of(ks, ks_log2, 4 * r4);
            if (vec) {
                if (own0 && i < dk) *reinterpret_cast<float4*>(scol0 + i) = make_float4(S0[4 * r4], S0[4 * r4 + 1], S0[4 * r4 + 2], S0[4 * r4 + 3]);
                if (own1 && i < dk) *reinterpret_cast<float4*>(scol1 + i) = make_float4(S1[4 * r4], S1[4 * r4 + 1], S1[4 * r4 + 2], S1[4 * r4 + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (own0 && i + j < dk) scol0[i + j] = S0[4 * r4 + j];
                    if (own1 && i + j < dk) scol1[i + j] = S1[4 * r4 + j];
                }
            }
        }
    }
}

// The decay of every key channel over a whole chunk: exp(-sum_t exp(dlog[t])) (the product of the tokens' decays),
// the product of sigmoid(dlog[t])^sigmoid_power where that power is given,
// or decay_h ^ tokens for a fixed decay per head.  chunk_decay [chunks][H * dk].
__global__ void chunk_decay_kernel(float* __restrict__ chunk_decay, const float* __restrict__ dlog, size_t ldd,
                                   const float* __restrict__ head_decay, const int32_t* __restrict__ chunk_start,
                                   int n, int dk, const float* __restrict__ ga, size_t ldg, float sigmoid_power) {
    const int c = blockIdx.x;
    const int t0 = chunk_start[c], t1 = chunk_start[c + 1];
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < n; i += gridDim.y * blockDim.x) {
        float a;
        if (dlog && sigmoid_power > 0.f) {              // w = sigmoid(z)^power per token: the product, token by token
            a = 1.0f;
            for (int t = t0; t < t1; ++t) a *= expf(log_sigmoid_f32(dlog[(size_t)t * ldd + i]) * sigmoid_power);
        } else if (dlog) {
            float sum = 0.f;
            for (int t = t0; t < t1; ++t) sum += expf(dlog[(size_t)t * ldd + i]);
            a = expf(-sum);
        } else if (ga) {                                // a decay per token and head: their product in order
            a = 1.0f;
            for (int t = t0; t < t1; ++t) a *= ga[(size_t)t * ldg + i / dk];
        } else {
            a = 1.0f;
            const float d = head_decay[i / dk];
            for (int t = t0; t < t1; ++t) a *= d;
        }
        chunk_decay[(size_t)c * n + i] = a;
    }
}

// Walk each sequence's chunks in order: chunk_state[c] (what chunk c adds, from PHASE 1) becomes the state that
// chunk c starts from; the state after the last chunk goes to the sequence's slot.  One thread per state element
// [h][j][i]; the decay belongs to (h, i).
__global__ void chunk_prefix_kernel(float* __restrict__ chunk_state, const float* __restrict__ chunk_decay,
                                    float* __restrict__ state, size_t slot_stride, const int32_t* __restrict__ seq_chunk,
                                    const int32_t* __restrict__ seq_slot, int H, int dk, int dv) {
    const int s = blockIdx.x;
    const int slot = seq_slot[s];
    const int c0 = seq_chunk[s], c1 = seq_chunk[s + 1];
    if (slot < 0 || c1 <= c0) return;
    const size_t n = (size_t)H * dv * dk;
    constexpr int AHEAD = 8;                            // chunks whose loads are in flight together
    for (size_t e = (size_t)blockIdx.y * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.y * blockDim.x) {
        const int i = (int)(e % dk), h = (int)(e / ((size_t)dv * dk));
        const float* dec = chunk_decay + (size_t)h * dk + i;
        float S = state[(size_t)slot * slot_stride + e];
        for (int c = c0; c < c1; c += AHEAD) {
            float added[AHEAD], a[AHEAD];
#pragma unroll
            for (int g = 0; g < AHEAD; ++g) {
                added[g] = c + g < c1 ? chunk_state[(size_t)(c + g) * n + e] : 0.f;
                a[g] = c + g < c1 ? dec[(size_t)(c + g) * H * dk] : 1.f;
            }
#pragma unroll
            for (int g = 0; g < AHEAD; ++g) {
                if (c + g < c1) {
                    chunk_state[(size_t)(c + g) * n + e] = S;
                    S = fmaf(a[g], S, added[g]);
                }
            }
        }
        state[(size_t)slot * slot_stride + e] = S;
    }
}

// ----------------------------------------------------------------------------- token shift

// out[m][t] = h[t] + (h[t-1] - h[t]) * mu[m], m < n_mix; h[t-1] is zero for a sequence's first token, the row
// above inside a step, and what the earlier steps left in `last_row[slot]` for the first row of a later step.
template <typename T>
__global__ void token_shift_kernel(T* __restrict__ out, size_t ldo, size_t mix_stride, const T* __restrict__ h, size_t ldh,
                                   const float* __restrict__ mu, const T* __restrict__ last_row, size_t ld_last,
                                   const int32_t* __restrict__ tok_slot, const int32_t* __restrict__ tok_pos,
                                   int D, int n_mix) {
    grid_dep_launch();
    grid_dep_wait();
    const int t = blockIdx.x;
    const int slot = tok_slot[t];
    const T* before = nullptr;
    if (slot >= 0 && tok_pos[t] > 0)
        before = (t > 0 && tok_slot[t - 1] == slot) ? h + (size_t)(t - 1) * ldh : last_row + (size_t)slot * ld_last;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const float cur = slot >= 0 ? to_f32(h[(size_t)t * ldh + i]) : 0.f;
        const float diff = (before ? to_f32(before[i]) : 0.f) - cur;
        for (int m = 0; m < n_mix; ++m)
            out[(size_t)m * mix_stride + (size_t)t * ldo + i] = from_f32<T>(fmaf(diff, mu[(size_t)m * D + i], cur));
    }
}

// The delta rule over chunks that ran side by side.  A chunk's tokens act on the state as S <- P S + Q, with
// P = A_n .. A_1 (A_t = (I - beta_t k_t k_t^T) diag(g_t), the same for every value column) and Q what the chunk
// writes from an empty state; both come from the scan itself (P: the scan of an identity with values of zero).  This
// kernel walks a sequence's chunks in order: it leaves in `start` the state each chunk starts from and in the slot the
// state after the last.  Layouts as the state's: P [chunks][H][dk (column j)][dk (row i)], Q and start
// [chunks][H][dv][dk].  A block owns DCB value columns of one head; nothing is divided by a decay, so small decays
// cost no precision.
constexpr int DCB = 16;
__global__ void __launch_bounds__(128)
delta_chunk_prefix_kernel(const float* __restrict__ P, const float* __restrict__ Q, float* __restrict__ start,
                          float* __restrict__ state, size_t slot_stride, const int32_t* __restrict__ seq_chunk,
                          const int32_t* __restrict__ seq_slot, int H, int dk, int dv) {
    extern __shared__ float s_cur[];                    // [dk][DCB]: the state's rows of this block's columns
    grid_dep_launch();
    grid_dep_wait();
    const int s = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * DCB;
    const int slot = seq_slot[s];
    if (slot < 0) return;
    const int n_cols = min(DCB, dv - col0);
    float* mine = state + (size_t)slot * slot_stride + ((size_t)h * dv + col0) * dk;
    for (int e = threadIdx.x; e < DCB * dk; e += blockDim.x) {
        const int c = e / dk, i = e - c * dk;
        s_cur[i * DCB + c] = c < n_cols ? mine[(size_t)c * dk + i] : 0.f;
    }
    for (int ch = seq_chunk[s]; ch < seq_chunk[s + 1]; ++ch) {
        __syncthreads();
        float* st = start + (((size_t)ch * H + h) * dv + col0) * dk;
        for (int e = threadIdx.x; e < n_cols * dk; e += blockDim.x) {
            const int c = e / dk, i = e - c * dk;
            st[(size_t)c * dk + i] = s_cur[i * DCB + c];
        }
        const float* Pc = P + ((size_t)ch * H + h) * dk * dk;
        const float* Qc = Q + (((size_t)ch * H + h) * dv + col0) * dk;
        float acc[2][DCB];                              // rows threadIdx.x and threadIdx.x + 128 (dk is at most 256)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int i = threadIdx.x + r * 128;
#pragma unroll
            for (int c = 0; c < DCB; ++c) acc[r][c] = (i < dk && c < n_cols) ? Qc[(size_t)c * dk + i] : 0.f;
        }
        for (int j = 0; j < dk; ++j) {
            const float p0 = threadIdx.x < dk ? Pc[(size_t)j * dk + threadIdx.x] : 0.f;
            const float p1 = threadIdx.x + 128 < dk ? Pc[(size_t)j * dk + threadIdx.x + 128] : 0.f;
            const float4* row = reinterpret_cast<const float4*>(s_cur + j * DCB);
#pragma unroll
            for (int c4 = 0; c4 < DCB / 4; ++c4) {
                const float4 x = row[c4];
                acc[0][4 * c4] = fmaf(p0, x.x, acc[0][4 * c4]);         acc[1][4 * c4] = fmaf(p1, x.x, acc[1][4 * c4]);
                acc[0][4 * c4 + 1] = fmaf(p0, x.y, acc[0][4 * c4 + 1]); acc[1][4 * c4 + 1] = fmaf(p1, x.y, acc[1][4 * c4 + 1]);
                acc[0][4 * c4 + 2] = fmaf(p0, x.z, acc[0][4 * c4 + 2]); acc[1][4 * c4 + 2] = fmaf(p1, x.z, acc[1][4 * c4 + 2]);
                acc[0][4 * c4 + 3] = fmaf(p0, x.w, acc[0][4 * c4 + 3]); acc[1][4 * c4 + 3] = fmaf(p1, x.w, acc[1][4 * c4 + 3]);
            }
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int i = threadIdx.x + r * 128;
            if (i < dk) {
#pragma unroll
                for (int c = 0; c < DCB; ++c) s_cur[i * DCB + c] = acc[r][c];
            }
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_cols * dk; e += blockDim.x) {
        const int c = e / dk, i = e - c * dk;
        mine[(size_t)c * dk + i] = s_cur[i * DCB + c];
    }
}

template <typename TI>
int launch_scan(int mode, int phase, float* o, long long ldo, const void* q, long long ldq, const void* k, long long ldk,
                const void* v, long long ldv, const float* dlog, long long ldd, const float* head_decay, const void* bonus,
                int bonus_dtype, float* state, long long slot_stride, const int32_t* seq_start, const int32_t* seq_slot,
                int n_seq, int T_rows, int H, int dk, int dv, int in_act, const float* ga, const float* gb, long long ldg,
                float q_scale, int qk_group, float decay_scale, cudaStream_t stream) {
    const bool wkv = mode == 1 || mode == 3 || mode == 4;            // a decay per token and key channel, staged beside q and k
    int ks_log2 = 0;
    while ((RK << ks_log2) < dk) ++ks_log2;
    const int KS = 1 << ks_log2;
    int cols = CPT * 256 / KS;
    if (cols > dv) cols = (dv + CPT - 1) / CPT * CPT;
    // the blocks of a head share its columns evenly: a count just above a block's width (a column more, as the gated
    // form has) would else leave a second block with a column or two and the whole staging to do for them
    { const int nb = (dv + cols - 1) / cols; cols = ((dv + nb - 1) / nb + CPT - 1) / CPT * CPT; }
    // few sequences and heads: narrower blocks, so that more SMs take part
    while (cols > 8 * CPT && (long long)n_seq * H * ((dv + cols - 1) / cols) < 148 && cols / CPT * KS > 64)
        cols = (cols / 2 + CPT - 1) / CPT * CPT;       // whole pairs of columns, also for an odd count
    const int threads = ((cols / CPT * KS + 31) / 32) * 32;
    const int dkp = KS * RK;
    const size_t smem = ((size_t)TILE * ((wkv ? 3 : 2) * dkp + cols) + dkp + TILE) * sizeof(float);
    const int vec = dk % 4 == 0 && slot_stride % 4 == 0 && ((uintptr_t)state % 16) == 0;
    dim3 grid(n_seq, H, (dv + cols - 1) / cols);
    cudaError_t e;
#define GO(MODE, PHASE) do { e = smem > 48 * 1024 ? cudaFuncSetAttribute(state_scan_kernel<TI, MODE, PHASE>, \
            cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) : cudaSuccess; \
    if (e == cudaSuccess) e = qs_launch_dependent(state_scan_kernel<TI, MODE, PHASE>, grid, dim3(threads), smem, stream, o, (size_t)ldo, \
        (const TI*)q, (size_t)ldq, (const TI*)k, (size_t)ldk, (const TI*)v, (size_t)ldv, dlog, (size_t)ldd, head_decay, bonus, \
        bonus_dtype, state, (size_t)slot_stride, seq_start, seq_slot, n_seq, T_rows, H, dk, dv, ks_log2, cols, in_act, vec, \
        ga, gb, (size_t)ldg, q_scale, qk_group, decay_scale); } while (0)
    if (mode == 3) GO(3, 0);
    else if (mode == 4) { if (phase == 0) GO(4, 0); else if (phase == 1) GO(4, 1); else GO(4, 3); }
    else if (mode == 1) { if (phase == 0) GO(1, 0); else if (phase == 1) GO(1, 1); else GO(1, 3); }
    else if (mode == 2) { if (phase == 0) GO(2, 0); else if (phase == 1) GO(2, 1); else GO(2, 3); }
    else { if (phase == 0) GO(0, 0); else if (phase == 1) GO(0, 1); else GO(0, 3); }
#undef GO
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "state_scan: %s", cudaGetErrorString(e));
    return qs_check_launch("state_scan");
}

// ----------------------------------------------------------------------------- mLSTM: gates and output

// The exponential gates of an mLSTM, stabilised by a running maximum m per sequence and head (0 for an empty
// sequence).  From the raw gate projections (bias included) raw [T, 2 H] = (input | forget):
//     i = cap tanh(raw_i / cap),  f = logsigmoid(cap tanh(raw_f / cap))          (cap 0: no cap)
//     m_t = max(f + m_{t-1}, i),  a_t = exp(f + m_{t-1} - m_t),  b_t = exp(i - m_t)
// One block per sequence of the step.  The transcendental functions of all its tokens and heads are taken side by
// side (i and f rest in the outputs meanwhile); only the chain of maxima, an addition and a maximum per token,
// runs in order, one thread per head; then a and b side by side again.  m is kept per slot.
__global__ void mlstm_gates_kernel(float* __restrict__ ga, float* __restrict__ gb, float* __restrict__ gm, size_t ldg,
                                   const float* __restrict__ raw, size_t ldr, float cap, float* __restrict__ m_state,
                                   size_t slot_stride, const int32_t* __restrict__ seq_start,
                                   const int32_t* __restrict__ seq_slot, int n_seq, int T_rows, int H) {
    grid_dep_launch();
    grid_dep_wait();
    const int s = blockIdx.x;
    if (s == n_seq) {                                   // rows that belong to nobody
        const int first = seq_start[n_seq];
        for (int e = threadIdx.x; e < (T_rows - first) * H; e += blockDim.x) {
            const size_t at = (size_t)(first + e / H) * ldg + e % H;
            ga[at] = 1.f; gb[at] = 0.f; gm[at] = 0.f;
        }
        return;
    }
    const int slot = seq_slot[s];
    const int t0 = seq_start[s], n = seq_start[s + 1] - t0;
    if (slot < 0) {
        for (int e = threadIdx.x; e < n * H; e += blockDim.x) {
            const size_t at = (size_t)(t0 + e / H) * ldg + e % H;
            ga[at] = 1.f; gb[at] = 0.f; gm[at] = 0.f;
        }
        return;
    }
    for (int e = threadIdx.x; e < n * H; e += blockDim.x) {
        const int t = t0 + e / H, h = e % H;
        float ri = raw[(size_t)t * ldr + h], rf = raw[(size_t)t * ldr + H + h];
        if (cap > 0.f) { ri = cap * tanhf(ri / cap); rf = cap * tanhf(rf / cap); }
        gb[(size_t)t * ldg + h] = ri;
        ga[(size_t)t * ldg + h] = log_sigmoid_f32(rf);
    }
    __syncthreads();
    constexpr int AHEAD = 8;                            // tokens whose loads are in flight together
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        float m = m_state[(size_t)slot * slot_stride + h];
        for (int base = 0; base < n; base += AHEAD) {
            float f[AHEAD], i[AHEAD];
#pragma unroll
            for (int j = 0; j < AHEAD; ++j) {
                const size_t at = (size_t)(t0 + min(base + j, n - 1)) * ldg + h;
                f[j] = ga[at]; i[j] = gb[at];
            }
#pragma unroll
            for (int j = 0; j < AHEAD; ++j)
                if (base + j < n) { m = fmaxf(f[j] + m, i[j]); gm[(size_t)(t0 + base + j) * ldg + h] = m; }
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n * H; e += blockDim.x) {
        const int t = t0 + e / H, h = e % H;
        const size_t at = (size_t)t * ldg + h;
        const float before = t == t0 ? m_state[(size_t)slot * slot_stride + h] : gm[at - ldg];
        const float m = gm[at];
        ga[at] = expf(ga[at] + before - m);
        gb[at] = expf(gb[at] - m);
    }
    __syncthreads();
    if (n > 0)
        for (int h = threadIdx.x; h < H; h += blockDim.x)
            m_state[(size_t)slot * slot_stride + h] = gm[(size_t)(t0 + n - 1) * ldg + h];
}

// The same in three kernels for steps with long sequences.  First the log gates of every row, side by side:
// ga <- f, gb <- i.
__global__ void mlstm_gate_logs_kernel(float* __restrict__ ga, float* __restrict__ gb, size_t ldg, const float* __restrict__ raw,
                                       size_t ldr, float cap, int T_rows, int H) {
    grid_dep_launch();
    grid_dep_wait();
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= (long long)T_rows * H) return;
    const int t = (int)(e / H), h = (int)(e % H);
    float ri = raw[(size_t)t * ldr + h], rf = raw[(size_t)t * ldr + H + h];
    if (cap > 0.f) { ri = cap * tanhf(ri / cap); rf = cap * tanhf(rf / cap); }
    gb[(size_t)t * ldg + h] = ri;
    ga[(size_t)t * ldg + h] = log_sigmoid_f32(rf);
}

// Then the chain of maxima, one warp per (sequence, head).  m -> max(m + f, i) composes: first (F1, I1), then
// (F2, I2) is (F1 + F2, max(I1 + F2, I2)).  A lane folds its run of consecutive tokens into one such pair, the
// lanes' pairs are scanned by shuffles, and each lane walks its run again from the maximum it starts with.  What
// the sequence held before goes to `m_before`, the last maximum to the slot.
__global__ void mlstm_gate_scan_kernel(float* __restrict__ gm, const float* __restrict__ ga, const float* __restrict__ gb,
                                       size_t ldg, float* __restrict__ m_state, size_t slot_stride, float* __restrict__ m_before,
                                       const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_slot, int H) {
    grid_dep_launch();
    grid_dep_wait();
    const int s = blockIdx.x, lane = threadIdx.x & 31;
    const int slot = seq_slot[s];
    const int t0 = seq_start[s], n = seq_start[s + 1] - t0;
    if (slot < 0 || n <= 0) return;
    const int run = (n + 31) / 32;
    const int a = min(n, lane * run), b = min(n, a + run);
    for (int h = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5); h < H; h += gridDim.y * (blockDim.x >> 5)) {
        const float m0 = m_state[(size_t)slot * slot_stride + h];
        float F = 0.f, I = -INFINITY;
        for (int t = a; t < b; ++t) {
            const float f = ga[(size_t)(t0 + t) * ldg + h], i = gb[(size_t)(t0 + t) * ldg + h];
            F += f;
            I = fmaxf(I + f, i);
        }
        // inclusive scan of the lanes' pairs, in lane order
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const float Fp = __shfl_up_sync(0xffffffffu, F, off), Ip = __shfl_up_sync(0xffffffffu, I, off);
            if (lane >= off) { I = fmaxf(Ip + F, I); F = Fp + F; }
        }
        // the maximum this lane's run starts with: m0 through the pairs of the lanes before it
        const float Fb = __shfl_up_sync(0xffffffffu, F, 1), Ib = __shfl_up_sync(0xffffffffu, I, 1);
        float m = lane == 0 ? m0 : fmaxf(m0 + Fb, Ib);
        for (int t = a; t < b; ++t) {
            m = fmaxf(ga[(size_t)(t0 + t) * ldg + h] + m, gb[(size_t)(t0 + t) * ldg + h]);
            gm[(size_t)(t0 + t) * ldg + h] = m;
        }
        const float last = __shfl_sync(0xffffffffu, fmaxf(m0 + F, I), 31);
        if (lane == 0) { m_before[(size_t)s * H + h] = m0; m_state[(size_t)slot * slot_stride + h] = last; }
    }
}

// Last the factors, side by side: a = exp(f + m_{t-1} - m_t), b = exp(i - m_t); rows of no sequence get a = 1, b = 0.
__global__ void mlstm_gate_factors_kernel(float* __restrict__ ga, float* __restrict__ gb, float* __restrict__ gm, size_t ldg,
                                          const float* __restrict__ m_before, const int32_t* __restrict__ seq_start,
                                          const int32_t* __restrict__ seq_slot, int n_seq, int T_rows, int H) {
    grid_dep_launch();
    grid_dep_wait();
    const int s = blockIdx.x;
    const int t0 = seq_start[s], n = (s == n_seq ? T_rows : seq_start[s + 1]) - t0;
    const bool live = s < n_seq && seq_slot[s] >= 0;
    for (long long e = (long long)blockIdx.y * blockDim.x + threadIdx.x; e < (long long)n * H; e += (long long)gridDim.y * blockDim.x) {
        const int t = (int)(e / H), h = (int)(e % H);
        const size_t at = (size_t)(t0 + t) * ldg + h;
        if (!live) { ga[at] = 1.f; gb[at] = 0.f; gm[at] = 0.f; continue; }
        const float before = t == 0 ? m_before[(size_t)s * H + h] : gm[at - ldg];
        const float m = gm[at];
        ga[at] = expf(ga[at] + before - m);
        gb[at] = expf(gb[at] - m);
    }
}

// What follows the recurrence: per token and head, o [dv] and the normaliser's product nq (the element behind o):
//     y = o / (max(|nq|, exp(-m)) + 1e-6);  y / sqrt(mean(y^2) + eps) * w * sigmoid(gate)
// One block per token, a warp per head in turn; sums in 32-bit in a fixed order.
template <typename TG, typename TO>
__global__ void mlstm_output_kernel(TO* __restrict__ out, size_t ldo, const float* __restrict__ o, size_t ldi,
                                    const float* __restrict__ gm, size_t ldg, const void* __restrict__ w, int w_dtype,
                                    const TG* __restrict__ gate, size_t ldgate, int H, int dv, float eps) {
    grid_dep_launch();
    grid_dep_wait();
    const size_t t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    for (int h = warp; h < H; h += warps) {
        const float* src = o + t * ldi + (size_t)h * (dv + 1);
        const float den = fmaxf(fabsf(src[dv]), expf(-gm[t * ldg + h])) + 1e-6f;
        float s = 0.f;
        for (int j = lane; j < dv; j += 32) { const float y = src[j] / den; s = fmaf(y, y, s); }
        const float rstd = 1.0f / sqrtf(warp_sum(s) / (float)dv + eps);
        for (int j = lane; j < dv; j += 32) {
            const size_t c = (size_t)h * dv + j;
            out[t * ldo + c] = from_f32<TO>(src[j] / den * rstd * load_as_f32(w, w_dtype, c) *
                                            sigmoid_f32(to_f32(gate[t * ldgate + c])));
        }
    }
}

}  // namespace

// `m_before` (n_seq * H floats of scratch, or null): with it, steps whose sequences are long on average take the gates
// in three kernels, the chain of maxima as a scan over each sequence; the results differ from the walk in order by
// rounding only.
QS_API int qs_mlstm_gates(float* ga, float* gb, float* gm, long long ldg, const float* raw, long long ldr, float cap,
                          float* m_state, long long slot_stride, const int32_t* seq_start, const int32_t* seq_slot,
                          int n_seq, int T_rows, int H, float* m_before, cudaStream_t stream) {
    if (T_rows == 0) return QS_OK;
    QS_REQUIRE(n_seq >= 0 && T_rows > 0 && H > 0 && cap >= 0.f, "mlstm_gates: bad sizes");
    if (m_before && n_seq > 0 && T_rows >= 128 * n_seq) {
        const long long total = (long long)T_rows * H;
        cudaError_t e = qs_launch_dependent(mlstm_gate_logs_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream,
                                            ga, gb, (size_t)ldg, raw, (size_t)ldr, cap, T_rows, H);
        if (e == cudaSuccess)
            e = qs_launch_dependent(mlstm_gate_scan_kernel, dim3(n_seq, (H + 3) / 4 > 64 ? 64 : (H + 3) / 4), dim3(128), 0, stream, gm,
                                    (const float*)ga, (const float*)gb, (size_t)ldg, m_state, (size_t)slot_stride, m_before,
                                    seq_start, seq_slot, H);
        if (e == cudaSuccess)
            e = qs_launch_dependent(mlstm_gate_factors_kernel, dim3(n_seq + 1, 32), dim3(256), 0, stream, ga, gb, gm, (size_t)ldg,
                                    (const float*)m_before, seq_start, seq_slot, n_seq, T_rows, H);
        if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "mlstm_gates: %s", cudaGetErrorString(e));
        return qs_check_launch("mlstm_gates");
    }
    const int threads = (long long)T_rows * H >= 4096 * (long long)(n_seq > 0 ? n_seq : 1) ? 512 : (T_rows * H > 64 * n_seq ? 128 : 32);
    cudaError_t e = qs_launch_dependent(mlstm_gates_kernel, dim3(n_seq + 1), dim3(threads), 0, stream, ga, gb, gm, (size_t)ldg,
                                        raw, (size_t)ldr, cap, m_state, (size_t)slot_stride, seq_start, seq_slot, n_seq,
                                        T_rows, H);
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "mlstm_gates: %s", cudaGetErrorString(e));
    return qs_check_launch("mlstm_gates");
}

QS_API int qs_mlstm_output(void* out, int out_dtype, long long ldo, const float* o, long long ldi, const float* gm,
                           long long ldg, const void* w, int w_dtype, const void* gate, int gate_dtype, long long ldgate,
                           int rows, int H, int dv, float eps, cudaStream_t stream) {
    if (rows == 0) return QS_OK;
    QS_REQUIRE(rows > 0 && H > 0 && dv > 0 && o && gm && w && gate, "mlstm_output: bad sizes or operands");
    const int threads = H >= 8 ? 256 : (H >= 4 ? 128 : 32 * H);
    typedef __nv_bfloat16 bf16;
    cudaError_t e;
#define GO(TG, TO) e = qs_launch_dependent(mlstm_output_kernel<TG, TO>, dim3(rows), dim3(threads), 0, stream, (TO*)out, (size_t)ldo, \
        o, (size_t)ldi, gm, (size_t)ldg, w, w_dtype, (const TG*)gate, (size_t)ldgate, H, dv, eps)
    if (gate_dtype == QS_F32 && out_dtype == QS_F32) GO(float, float);
    else if (gate_dtype == QS_BF16 && out_dtype == QS_BF16) GO(bf16, bf16);
    else if (gate_dtype == QS_BF16 && out_dtype == QS_F32) GO(bf16, float);
    else return qs_fail(QS_ERR_INVALID_INPUT, "mlstm_output: unsupported types gate=%d out=%d", gate_dtype, out_dtype);
#undef GO
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "mlstm_output: %s", cudaGetErrorString(e));
    return qs_check_launch("mlstm_output");
}

namespace {
}  // namespace

// mode 2: decay `ga` and input weight `gb` per token and head ([T, H] float32, `ldg` floats between rows), q times
// `q_scale`; dv counts one column more than v holds (the column of ones that carries the normaliser).
// mode 0: fixed decay per head (`head_decay` [H], float32 on the device); mode 1: decay exp(-exp(dlog)) per token and
// key channel (`dlog` [T, H * dk] float32) and the bonus `bonus` [H, dk] for the current token.
// q, k [T, H * dk] and v [T, H * dv] of type `dtype`, with `in_act` applied on the way in; o [T, H * dv] float32;
// state [slots][H][dv][dk] float32 with `slot_stride` floats between slots.
//
// With `chunk_start` (device, n_chunks + 1 rows of the packed batch; every sequence of the step cut into consecutive
// chunks, in packed order) the prompt's chunks run side by side: `seq_chunk` (n_seq + 1) names each sequence's
// chunks, `chunk_state` ([n_chunks][H][dv][dk]) and `chunk_decay` ([n_chunks][H * dk]) are scratch, `chunk_ids`
// holds 0 .. n_chunks - 1.  The result equals the walk in order up to the rounding of 32-bit sums.
QS_API int qs_state_scan(int mode, float* o, long long ldo, const void* q, long long ldq, const void* k, long long ldk,
                         const void* v, long long ldv, int dtype, const float* dlog, long long ldd, const float* head_decay,
                         const void* bonus, int bonus_dtype, float* state, long long slot_stride, const int32_t* seq_start,
                         const int32_t* seq_slot, int n_seq, int T_rows, int H, int dk, int dv, int in_act,
                         const int32_t* chunk_start, const int32_t* chunk_ids, int n_chunks, const int32_t* seq_chunk,
                         float* chunk_state, float* chunk_decay, const float* ga, const float* gb, long long ldg,
                         float q_scale, int qk_group, float decay_scale, cudaStream_t stream) {
    if (n_seq == 0 || T_rows == 0) return QS_OK;
    QS_REQUIRE(n_seq > 0 && T_rows > 0 && H > 0 && dk > 0 && dv > 0, "state_scan: bad sizes");
    QS_REQUIRE(dk <= 16 * RK, "state_scan: %d key channels per head above %d", dk, 16 * RK);
    QS_REQUIRE(H <= 65535, "state_scan: %d heads exceed the grid", H);
    QS_REQUIRE(mode == 0 ? head_decay != nullptr : mode == 1 ? (dlog && bonus) : mode == 2 ? (ga && gb && dv > 1)
               : mode == 4 ? (dlog && decay_scale > 0.f) : (mode == 3 && dlog && gb && !chunk_start),
               "state_scan: mode %d lacks its operands", mode);
    if (qk_group < 1) qk_group = 1;
    QS_REQUIRE(mode == 3 ? H % qk_group == 0 : qk_group == 1, "state_scan: %d heads in groups of %d", H, qk_group);
    QS_REQUIRE(dtype == QS_F32 || dtype == QS_BF16, "state_scan: unknown dtype %d", dtype);
    const bool wkv = mode == 1 || mode == 4;
    (void)wkv;
#define SCAN(PHASE, STATE, STRIDE, STARTS, SLOTS, N) (dtype == QS_F32 \
        ? launch_scan<float>(mode, PHASE, o, ldo, q, ldq, k, ldk, v, ldv, dlog, ldd, head_decay, bonus, bonus_dtype, STATE, STRIDE, \
                             STARTS, SLOTS, N, T_rows, H, dk, dv, in_act, ga, gb, ldg, q_scale, qk_group, decay_scale, stream) \
        : launch_scan<__nv_bfloat16>(mode, PHASE, o, ldo, q, ldq, k, ldk, v, ldv, dlog, ldd, head_decay, bonus, bonus_dtype, STATE, \
                                     STRIDE, STARTS, SLOTS, N, T_rows, H, dk, dv, in_act, ga, gb, ldg, q_scale, qk_group, decay_scale, stream))
    if (!chunk_start) return SCAN(0, state, slot_stride, seq_start, seq_slot, n_seq);
    QS_REQUIRE(n_chunks > 0 && chunk_ids && seq_chunk && chunk_state && chunk_decay, "state_scan: chunks without their scratch");
    const long long per_chunk = (long long)H * dv * dk;
    int rc = SCAN(1, chunk_state, per_chunk, chunk_start, chunk_ids, n_chunks);
    if (rc != QS_OK) return rc;
    const int n = H * dk;
    chunk_decay_kernel<<<dim3(n_chunks, (n + 127) / 128), 128, 0, stream>>>(chunk_decay, wkv ? dlog : nullptr, (size_t)ldd,
                                                                            head_decay, chunk_start, n, dk,
                                                                            mode == 2 ? ga : nullptr, (size_t)ldg,
                                                                            mode == 4 ? decay_scale : 0.f);
    if ((rc = qs_check_launch("state_scan chunk decay")) != QS_OK) return rc;
    int by = (int)((per_chunk + 255) / 256);
    if (by > 1024) by = 1024;
    chunk_prefix_kernel<<<dim3(n_seq, by), 256, 0, stream>>>(chunk_state, chunk_decay, state, (size_t)slot_stride, seq_chunk,
                                                              seq_slot, H, dk, dv);
    if ((rc = qs_check_launch("state_scan chunk prefix")) != QS_OK) return rc;
    return SCAN(3, chunk_state, per_chunk, chunk_start, chunk_ids, n_chunks);
#undef SCAN
}

// See delta_chunk_prefix_kernel.  seq_chunk (n_seq + 1) names each sequence's chunks; a sequence's slot must be a row
// of `state` (or negative: skipped).
QS_API int qs_delta_chunk_prefix(const float* P, const float* Q, float* start, float* state, long long slot_stride,
                                 const int32_t* seq_chunk, const int32_t* seq_slot, int n_seq, int H, int dk, int dv,
                                 cudaStream_t stream) {
    if (n_seq == 0) return QS_OK;
    QS_REQUIRE(n_seq > 0 && H > 0 && dk > 0 && dk <= 256 && dv > 0 && H <= 65535, "delta_chunk_prefix: bad sizes");
    const size_t smem = (size_t)dk * DCB * sizeof(float);
    cudaError_t e = qs_launch_dependent(delta_chunk_prefix_kernel, dim3(n_seq, H, (dv + DCB - 1) / DCB), dim3(128), smem, stream,
                                        P, Q, start, state, (size_t)slot_stride, seq_chunk, seq_slot, H, dk, dv);
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "delta_chunk_prefix: %s", cudaGetErrorString(e));
    return qs_check_launch("delta_chunk_prefix");
}

QS_API int qs_token_shift(void* out, long long ldo, long long mix_stride, const void* h, long long ldh, int dtype,
                          const float* mu, const void* last_row, long long ld_last, const int32_t* tok_slot,
                          const int32_t* tok_pos, int T, int D, int n_mix, cudaStream_t stream) {
    if (T == 0) return QS_OK;
    QS_REQUIRE(T > 0 && D > 0 && n_mix > 0, "token_shift: bad sizes");
    const int threads = D >= 1024 ? 256 : 128;
    cudaError_t e;
    if (dtype == QS_F32)
        e = qs_launch_dependent(token_shift_kernel<float>, dim3(T), dim3(threads), 0, stream, (float*)out, (size_t)ldo,
                                (size_t)mix_stride, (const float*)h, (size_t)ldh, mu, (const float*)last_row, (size_t)ld_last,
                                tok_slot, tok_pos, D, n_mix);
    else if (dtype == QS_BF16)
        e = qs_launch_dependent(token_shift_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, (__nv_bfloat16*)out,
                                (size_t)ldo, (size_t)mix_stride, (const __nv_bfloat16*)h, (size_t)ldh, mu,
                                (const __nv_bfloat16*)last_row, (size_t)ld_last, tok_slot, tok_pos, D, n_mix);
    else return qs_fail(QS_ERR_INVALID_INPUT, "token_shift: unknown dtype %d", dtype);
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "token_shift: %s", cudaGetErrorString(e));
    return qs_check_launch("token_shift");
}
