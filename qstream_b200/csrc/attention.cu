// Rotary position encoding fused with the write of keys and values into the paged
// cache, and causal attention of each token over its sequence's cache.
//
// Cache entry layout: K [n_pages][n_kv_heads][page_tokens][head_dim], V the same with the values' head size
// (dv, which may differ from the keys').
// A sequence (slot) owns a row of `page_table` ([n_slots][max_pages], int32); position
// p of the sequence lies in page page_table[slot][p / page_tokens] at row
// p % page_tokens.  A token with slot < 0 is padding: nothing is read or written for it.
#include "common.cuh"

namespace {

// ----------------------------------------------------------------------------- rotary + store

// For every token and head: rotate pairs (2j, 2j+1), 2j < R, of q (in place) and k by the
// angle pos * base^(-2j/R), taken from a 32-bit table [max_pos][R/2][2] = (cos, sin):
//   a' = a cos - b sin ; b' = a sin + b cos            (QStream src/engine.c:216-218)
// then keep the rotated k and the v in the cache (rope before store: src/engine.c:871-880).
// The rotation is evaluated in 32-bit and rounded once.  q == nullptr: keys/values only.
template <typename T>
__global__ void rope_store_kernel(T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                                  size_t ldq, size_t ldk, size_t ldv,
                                  int n_heads, int n_kv_heads, int dh, int R,
                                  const float* __restrict__ cos_sin, int max_pos,
                                  const int32_t* __restrict__ tok_slot, const int32_t* __restrict__ tok_pos,
                                  const int32_t* __restrict__ page_table, int max_pages, int page_shift,
                                  T* __restrict__ k_cache, T* __restrict__ v_cache,
                                  int32_t* __restrict__ status, int dv, const T* __restrict__ v_first, size_t ldvf,
                                  float lam, int half_layout) {
    // blockIdx.x = token; the gridDim.y blocks of a token share its (head, pair of dims) items of q, then k and v
    // half_layout: the rotated pairs are (j, j + R/2) instead of (2j, 2j+1); the angles are the same
    grid_dep_launch();
    grid_dep_wait();
    const int t = blockIdx.x;
    const int tid = blockIdx.y * blockDim.x + threadIdx.x, stride = gridDim.y * blockDim.x;
    const int slot = tok_slot[t];
    if (slot < 0) return;
    const int pos = tok_pos[t];
    const int page_tokens = 1 << page_shift;
    const bool rotate = cos_sin != nullptr && R > 0;
    if (rotate && (pos < 0 || pos >= max_pos)) { if (threadIdx.x == 0) atomicExch(status, 1); return; }
    const float* cs = rotate ? cos_sin + (size_t)pos * R : nullptr;      // R/2 pairs of (cos, sin)
    const int half = dh >> 1;

    if (q && rotate) {
        const int rp = R >> 1;                                           // rotated pairs per head
        for (int e = tid; e < n_heads * rp; e += stride) {
            const int head = e / rp, j = e - head * rp;
            T* row = q + (size_t)t * ldq + (size_t)head * dh;
            const float c = cs[2 * j], sn = cs[2 * j + 1];
            const int ia = half_layout ? j : 2 * j, ib = half_layout ? j + rp : 2 * j + 1;
            const float a = to_f32(row[ia]), b = to_f32(row[ib]);
            row[ia] = from_f32<T>(a * c - b * sn);
            row[ib] = from_f32<T>(a * sn + b * c);
        }
    }
    if (n_kv_heads == 0) return;
    const int page = page_table[(size_t)slot * max_pages + (pos >> page_shift)];
    if (page < 0) { if (threadIdx.x == 0) atomicExch(status, 2); return; }
    const size_t in_page = (size_t)(pos & (page_tokens - 1));
    for (int e = tid; e < n_kv_heads * half; e += stride) {
        const int kvh = e / half, j = e - kvh * half;
        const size_t dst_off = (((size_t)page * n_kv_heads + kvh) * page_tokens + in_page) * dh;
        const T* krow = k + (size_t)t * ldk + (size_t)kvh * dh;
        T* kdst = k_cache + dst_off;
        if (half_layout) {                  // item j: the pair (j, j + R/2) while j < R/2, then two plain elements
            const int rp = rotate ? R >> 1 : 0;
            if (j < rp) {
                const float c = cs[2 * j], sn = cs[2 * j + 1];
                const float a = to_f32(krow[j]), b = to_f32(krow[j + rp]);
                kdst[j] = from_f32<T>(a * c - b * sn);
                kdst[j + rp] = from_f32<T>(a * sn + b * c);
            } else {
                kdst[2 * j] = krow[2 * j];
                kdst[2 * j + 1] = krow[2 * j + 1];
            }
        } else if (rotate && 2 * j < R) {
            const float c = cs[2 * j], sn = cs[2 * j + 1];
            const float a = to_f32(krow[2 * j]), b = to_f32(krow[2 * j + 1]);
            kdst[2 * j] = from_f32<T>(a * c - b * sn);
            kdst[2 * j + 1] = from_f32<T>(a * sn + b * c);
        } else {
            kdst[2 * j] = krow[2 * j];
            kdst[2 * j + 1] = krow[2 * j + 1];
        }
    }
    // values: kept as they are, or blended with another layer's values of the same token,
    // (1 - lam) v + lam v_first, in 32-bit and rounded once
    for (int e = tid; e < n_kv_heads * dv; e += stride) {
        const int kvh = e / dv, j = e - kvh * dv;
        const size_t dst_off = (((size_t)page * n_kv_heads + kvh) * page_tokens + in_page) * dv;
        const T val = v[(size_t)t * ldv + (size_t)kvh * dv + j];
        v_cache[dst_off + j] = v_first ? from_f32<T>((1.0f - lam) * to_f32(val) + lam * to_f32(v_first[(size_t)t * ldvf + (size_t)kvh * dv + j]))
                                       : val;
    }
}

// One RMS norm over a token's whole q row (all heads at once) and one over its whole k row, then the rotation and the
// cache write, in one pass: q[i] <- rot(q[i] * rstd_q * wq[i]) in place, the cache keeps rot(k[i] * rstd_k * wk[i]) and
// the values as they are (v may be k itself: values that are the keys as projected).  One block per token; statistics,
// weights and rotation in 32-bit, every result rounded once.  Rows of no sequence (slot < 0) get zeros.
template <typename T>
__global__ void norm_rope_store_kernel(T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                                       size_t ldq, size_t ldk, size_t ldv, const void* __restrict__ wq, int wq_dtype,
                                       const void* __restrict__ wk, int wk_dtype, float eps,
                                       int n_heads, int n_kv_heads, int dh, int dv, int R,
                                       const float* __restrict__ cos_sin, int max_pos,
                                       const int32_t* __restrict__ tok_slot, const int32_t* __restrict__ tok_pos,
                                       const int32_t* __restrict__ page_table, int max_pages, int page_shift,
                                       T* __restrict__ k_cache, T* __restrict__ v_cache, int32_t* __restrict__ status,
                                       int half_layout) {
    __shared__ float scratch[33];
    grid_dep_launch();
    grid_dep_wait();
    const int t = blockIdx.x, tid = threadIdx.x, stride = blockDim.x;
    const int slot = tok_slot[t];
    const int nq = n_heads * dh, nk = n_kv_heads * dh;
    T* qrow = q + (size_t)t * ldq;
    if (slot < 0) {
        for (int i = tid; i < nq; i += stride) qrow[i] = from_f32<T>(0.f);
        return;
    }
    const int pos = tok_pos[t];
    const bool rotate = cos_sin != nullptr && R > 0;
    if (rotate && (pos < 0 || pos >= max_pos)) { if (tid == 0) atomicExch(status, 1); return; }
    const float* cs = rotate ? cos_sin + (size_t)pos * R : nullptr;
    const T* krow = k + (size_t)t * ldk;
    float sq = 0.f, sk = 0.f;
    for (int i = tid; i < nq; i += stride) { const float x = to_f32(qrow[i]); sq = fmaf(x, x, sq); }
    for (int i = tid; i < nk; i += stride) { const float x = to_f32(krow[i]); sk = fmaf(x, x, sk); }
    const float rq = 1.0f / sqrtf(block_sum(sq, scratch) / (float)nq + eps);
    const float rk = nk > 0 ? 1.0f / sqrtf(block_sum(sk, scratch) / (float)nk + eps) : 0.f;
    const int half = dh >> 1, rp = rotate ? R >> 1 : 0;
    // an item is a pair of elements of one head: a rotated pair while j < R/2, then two plain neighbours
    for (int e = tid; e < n_heads * half; e += stride) {
        const int head = e / half, j = e - head * half;
        const bool turn = j < rp;
        const int ia = head * dh + ((turn && half_layout) ? j : 2 * j), ib = head * dh + ((turn && half_layout) ? j + rp : 2 * j + 1);
        const float a = to_f32(qrow[ia]) * rq * load_as_f32(wq, wq_dtype, ia), b = to_f32(qrow[ib]) * rq * load_as_f32(wq, wq_dtype, ib);
        const float c = turn ? cs[2 * j] : 1.f, sn = turn ? cs[2 * j + 1] : 0.f;
        qrow[ia] = from_f32<T>(a * c - b * sn);
        qrow[ib] = from_f32<T>(a * sn + b * c);
    }
    if (n_kv_heads == 0) return;
    const int page = page_table[(size_t)slot * max_pages + (pos >> page_shift)];
    if (page < 0) { if (tid == 0) atomicExch(status, 2); return; }
    const int page_tokens = 1 << page_shift;
    const size_t in_page = (size_t)(pos & (page_tokens - 1));
    for (int e = tid; e < n_kv_heads * half; e += stride) {
        const int kvh = e / half, j = e - kvh * half;
        const bool turn = j < rp;
        const int la = (turn && half_layout) ? j : 2 * j, lb = (turn && half_layout) ? j + rp : 2 * j + 1;
        const int ia = kvh * dh + la, ib = kvh * dh + lb;
        const float a = to_f32(krow[ia]) * rk * load_as_f32(wk, wk_dtype, ia), b = to_f32(krow[ib]) * rk * load_as_f32(wk, wk_dtype, ib);
        const float c = turn ? cs[2 * j] : 1.f, sn = turn ? cs[2 * j + 1] : 0.f;
        T* kdst = k_cache + (((size_t)page * n_kv_heads + kvh) * page_tokens + in_page) * dh;
        kdst[la] = from_f32<T>(a * c - b * sn);
        kdst[lb] = from_f32<T>(a * sn + b * c);
    }
    for (int e = tid; e < n_kv_heads * dv; e += stride) {
        const int kvh = e / dv, j = e - kvh * dv;
        v_cache[(((size_t)page * n_kv_heads + kvh) * page_tokens + in_page) * dv + j] = v[(size_t)t * ldv + (size_t)kvh * dv + j];
    }
}

// The same for bfloat16 with 16-byte accesses: an item is eight consecutive dims (four rotary pairs).
// Needs head size and rotary width multiples of 8 and 16-byte aligned rows.
__device__ __forceinline__ uint4 rotate8(const uint4 raw, const float* __restrict__ cs8) {
    // cs8: (cos, sin) of the four pairs, eight floats
    const float4 a = reinterpret_cast<const float4*>(cs8)[0], b = reinterpret_cast<const float4*>(cs8)[1];
    const float c[4] = {a.x, a.z, b.x, b.z}, sn[4] = {a.y, a.w, b.y, b.w};
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float x = __uint_as_float(w[i] << 16), y = __uint_as_float(w[i] & 0xffff0000u);
        const __nv_bfloat162 r = __floats2bfloat162_rn(x * c[i] - y * sn[i], x * sn[i] + y * c[i]);
        o[i] = *reinterpret_cast<const uint32_t*>(&r);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

__global__ void rope_store_vec_kernel(__nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                      const __nv_bfloat16* __restrict__ v, size_t ldq, size_t ldk, size_t ldv,
                                      int n_heads, int n_kv_heads, int dh, int R,
                                      const float* __restrict__ cos_sin, int max_pos,
                                      const int32_t* __restrict__ tok_slot, const int32_t* __restrict__ tok_pos,
                                      const int32_t* __restrict__ page_table, int max_pages, int page_shift,
                                      __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                      int32_t* __restrict__ status, int settled, int dv,
                                      const __nv_bfloat16* __restrict__ v_first, size_t ldvf, float lam) {
    grid_dep_launch();
    // `settled`: the step's slots, positions and pages and the table of angles were complete before the
    // previous kernel of the stream began.  Then they are fetched (the table's row only as far as L2) while
    // that kernel still runs.
    if (!settled) grid_dep_wait();
    const int t = blockIdx.x;
    const int tid = blockIdx.y * blockDim.x + threadIdx.x, stride = gridDim.y * blockDim.x;
    const int slot = tok_slot[t];
    const int pos = tok_pos[t];
    const bool rotate = cos_sin != nullptr && R > 0;
    const bool pos_ok = !rotate || (pos >= 0 && pos < max_pos);
    const float* cs = rotate && pos_ok ? cos_sin + (size_t)pos * R : nullptr;
    int page = -1;
    if (slot >= 0 && n_kv_heads > 0 && pos >= 0 && (pos >> page_shift) < max_pages)
        page = page_table[(size_t)slot * max_pages + (pos >> page_shift)];
    if (cs && slot >= 0 && threadIdx.x * 32 < R)
        asm volatile("prefetch.global.L2 [%0];" :: "l"(cs + threadIdx.x * 32));
    if (settled) grid_dep_wait();
    if (slot < 0) return;
    const int page_tokens = 1 << page_shift;
    if (!pos_ok) { if (threadIdx.x == 0) atomicExch(status, 1); return; }
    const int rc = R >> 3, hc = dh >> 3;                                 // 16-byte chunks of the rotary part / of a head
    if (q && rotate) {
        for (int e = tid; e < n_heads * rc; e += stride) {
            const int head = e / rc, c = e - head * rc;
            uint4* p = reinterpret_cast<uint4*>(q + (size_t)t * ldq + (size_t)head * dh + c * 8);
            *p = rotate8(*p, cs + c * 8);
        }
    }
    if (n_kv_heads == 0) return;
    if (page < 0) { if (threadIdx.x == 0) atomicExch(status, 2); return; }
    const size_t in_page = (size_t)(pos & (page_tokens - 1));
    if (dv == dh && !v_first) {             // values as wide as keys and kept as they are: one item moves a chunk of each
        for (int e = tid; e < n_kv_heads * hc; e += stride) {
            const int kvh = e / hc, c = e - kvh * hc;
            const size_t dst = (((size_t)page * n_kv_heads + kvh) * page_tokens + in_page) * dh + c * 8;
            uint4 kk = *reinterpret_cast<const uint4*>(k + (size_t)t * ldk + (size_t)kvh * dh + c * 8);
            if (rotate && c < rc) kk = rotate8(kk, cs + c * 8);
            *reinterpret_cast<uint4*>(k_cache + dst) = kk;
            *reinterpret_cast<uint4*>(v_cache + dst) = *reinterpret_cast<const uint4*>(v + (size_t)t * ldv + (size_t)kvh * dh + c * 8);
        }
        return;
    }
    const int vc = dv >> 3;                                              // 16-byte chunks of a head's values
    for (int e = tid; e < n_kv_heads * (hc + vc); e += stride) {
        const int kvh = e / (hc + vc), c = e - kvh * (hc + vc);
        const size_t row = ((size_t)page * n_kv_heads + kvh) * page_tokens + in_page;
        if (c < hc) {
            uint4 kk = *reinterpret_cast<const uint4*>(k + (size_t)t * ldk + (size_t)kvh * dh + c * 8);
            if (rotate && c < rc) kk = rotate8(kk, cs + c * 8);
            *reinterpret_cast<uint4*>(k_cache + row * dh + c * 8) = kk;
        } else {
            const int cv = c - hc;
            uint4 vv = *reinterpret_cast<const uint4*>(v + (size_t)t * ldv + (size_t)kvh * dv + cv * 8);
            if (v_first) {              // (1 - lam) v + lam v_first in 32-bit, rounded once
                const uint4 ff = *reinterpret_cast<const uint4*>(v_first + (size_t)t * ldvf + (size_t)kvh * dv + cv * 8);
                const uint32_t a[4] = {vv.x, vv.y, vv.z, vv.w}, b[4] = {ff.x, ff.y, ff.z, ff.w};
                uint32_t o[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float x0 = __uint_as_float(a[i] << 16), x1 = __uint_as_float(a[i] & 0xffff0000u);
                    const float y0 = __uint_as_float(b[i] << 16), y1 = __uint_as_float(b[i] & 0xffff0000u);
                    const __nv_bfloat162 r = __floats2bfloat162_rn((1.0f - lam) * x0 + lam * y0, (1.0f - lam) * x1 + lam * y1);
                    o[i] = *reinterpret_cast<const uint32_t*>(&r);
                }
                vv = make_uint4(o[0], o[1], o[2], o[3]);
            }
            *reinterpret_cast<uint4*>(v_cache + row * dv + cv * 8) = vv;
        }
    }
}

// ----------------------------------------------------------------------------- attention

// One warp per (token, query head).  Keys are visited 32 at a time in position order:
// lane l scores key base+l (s = q.k / sqrt(dh), QStream src/engine.c:888-906), the
// running maximum and sum are updated (softmax with max subtraction,
// src/kernels_scalar.c:188-213, in its streaming form) and the 32 weighted values are
// added in key order (src/engine.c:913-922).  Scores, maximum, exponentials, sum and
// the output accumulator are 32-bit.  The order of the sums depends only on the
// token's own position, never on the batch or on where the pages lie.
// Lane l owns output dims l, l+32, ...: NACC = ceil(dv / 32) accumulators (dv: the values' head size).
// softcap > 0: s <- softcap * tanh(s / softcap) before the softmax.
// Which keys a query at position p sees: first .. p, where first = p - window + 1 (window > 0), or the start of
// p's chunk (chunk > 0: chunks of that many positions counted from 0), or 0; and, with keep_first > 0, the keys
// 0 .. keep_first - 1 below `first` as well.  sink: one number per query head whose exponential joins the softmax's
// denominator without a key or a value.  maps > 1: a key row holds `maps` keys of dh side by side; query head j
// reads key number j % maps of key head (j / maps) / (heads per key head), and that key head's values.
// TO: the type of the result (that of q and the cache, or 32-bit where a later kernel still works on it).
template <typename T, int NACC, typename TO>
__global__ void __launch_bounds__(128)
attention_kernel(TO* __restrict__ out, const T* __restrict__ q, size_t ldo, size_t ldq,
                 const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                 const int32_t* __restrict__ page_table, int max_pages, int page_shift,
                 const int32_t* __restrict__ tok_slot, const int32_t* __restrict__ tok_pos,
                 int T_tokens, int n_heads, int n_kv_heads, int dh, float scale, int window,
                 int32_t* __restrict__ status, int dv, float softcap, int chunk, int keep_first,
                 const float* __restrict__ sink, int maps) {
    extern __shared__ float q_smem[];               // [warps][dh]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int warps = blockDim.x >> 5;
    const long long item = (long long)blockIdx.x * warps + warp;
    if (item >= (long long)T_tokens * n_heads) return;
    const int t = (int)(item / n_heads), head = (int)(item % n_heads);
    TO* o = out + (size_t)t * ldo + (size_t)head * dv;
    const int slot = tok_slot[t];
    if (slot < 0) {                                 // padding: defined output, no cache access
        for (int d = lane; d < dv; d += 32) o[d] = from_f32<TO>(0.f);
        return;
    }
    const int pos = tok_pos[t];
    const int kvh = (head / maps) / (n_heads / maps / n_kv_heads);  // QStream src/engine.c:884,889
    const int krow_width = dh * maps, k_off = (head % maps) * dh;
    const int page_tokens = 1 << page_shift;
    const int32_t* pages = page_table + (size_t)slot * max_pages;

    float* qs = q_smem + (size_t)warp * dh;
    const T* qrow = q + (size_t)t * ldq + (size_t)head * dh;
    for (int d = lane; d < dh; d += 32) qs[d] = to_f32(qrow[d]);
    __syncwarp();

    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    const int first = window > 0 ? max(0, pos - window + 1) : (chunk > 0 ? pos - pos % chunk : 0);
    const int kept = min(keep_first, first);        // keys 0 .. kept - 1 are seen besides first .. pos

    for (int seg = kept > 0 ? 0 : 1; seg < 2; ++seg) {
    const int seg_lo = seg == 0 ? 0 : first, seg_hi = seg == 0 ? kept : pos + 1;
    for (int base = seg_lo; base < seg_hi; base += 32) {
        const int key = base + lane;
        const bool live = key < seg_hi;
        float s = -INFINITY;
        const T* vrow = nullptr;
        if (live) {
            const int page = pages[key >> page_shift];
            if (page < 0) { atomicExch(status, 3); }
            else {
                const size_t off = ((size_t)page * n_kv_heads + kvh) * page_tokens + (key & (page_tokens - 1));
                const T* krow = k_cache + off * krow_width + k_off;
                vrow = v_cache + off * dv;
                float dot = 0.f;
                for (int d = 0; d < dh; ++d) dot = fmaf(qs[d], to_f32(krow[d]), dot);
                s = dot * scale;
                if (softcap > 0.f) s = softcap * tanhf(s / softcap);
            }
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = live && vrow ? expf(s - m_new) : 0.f;
        const float alpha = m == -INFINITY ? 0.f : expf(m - m_new);
        l = l * alpha + warp_sum(p);
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[i] *= alpha;
        const int n_keys = min(32, seg_hi - base);
        for (int j = 0; j < n_keys; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const T* vj = reinterpret_cast<const T*>(__shfl_sync(0xffffffffu, (unsigned long long)vrow, j));
            if (!vj) continue;
#pragma unroll
            for (int i = 0; i < NACC; ++i) {
                const int d = lane + 32 * i;
                if (d < dv) acc[i] = fmaf(pj, to_f32(vj[d]), acc[i]);
            }
        }
        m = m_new;
    }
    }
    if (sink) {
        const float sk = sink[head];
        const float m_new = fmaxf(m, sk);
        const float alpha = m == -INFINITY ? 0.f : expf(m - m_new);
        l = l * alpha + expf(sk - m_new);
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[i] *= alpha;
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
        const int d = lane + 32 * i;
        if (d < dv) o[d] = from_f32<TO>(acc[i] * inv);
    }
}

template <typename T, typename TO>
int launch_attention(void* out, const void* q, long long ldo, long long ldq, const void* k_cache,
                     const void* v_cache, const int32_t* page_table, int max_pages, int page_shift,
                     const int32_t* tok_slot, const int32_t* tok_pos, int T_tokens, int n_heads,
                     int n_kv_heads, int dh, float scale, int window, int32_t* status, int dv, float softcap,
                     int chunk, int keep_first, const float* sink, int maps, cudaStream_t stream) {
    const int warps = 4;
    const long long items = (long long)T_tokens * n_heads;
    const int blocks = (int)((items + warps - 1) / warps);
    const size_t smem = (size_t)warps * dh * sizeof(float);
#define GO(NACC) attention_kernel<T, NACC, TO><<<blocks, warps * 32, smem, stream>>>( \
        (TO*)out, (const T*)q, (size_t)ldo, (size_t)ldq, (const T*)k_cache, (const T*)v_cache, \
        page_table, max_pages, page_shift, tok_slot, tok_pos, T_tokens, n_heads, n_kv_heads, dh, \
        scale, window, status, dv, softcap, chunk, keep_first, sink, maps)
    const int nacc = (dv + 31) / 32;
    if (nacc <= 1) GO(1);
    else if (nacc <= 2) GO(2);
    else if (nacc <= 4) GO(4);
    else if (nacc <= 8) GO(8);
    else GO(16);
#undef GO
    return qs_check_launch("attention");
}

}  // namespace

// `settled` != 0: slots, positions, page table and the table of angles were complete before the previous kernel
// of the stream began (they came by a copy, or from an earlier step), so the kernel may read them early.
QS_API int qs_rope_store(void* q, const void* k, const void* v, int dtype,
                         long long ldq, long long ldk, long long ldv,
                         int n_heads, int n_kv_heads, int dh, int R,
                         const float* cos_sin, int max_pos,
                         const int32_t* tok_slot, const int32_t* tok_pos,
                         const int32_t* page_table, int max_pages, int page_tokens,
                         void* k_cache, void* v_cache, int T_tokens, int32_t* status,
                         int settled, int dv, const void* v_first, long long ldvf, float lam, int half_layout,
                         cudaStream_t stream) {
    if (T_tokens == 0) return QS_OK;
    if (dv <= 0) dv = dh;
    QS_REQUIRE(T_tokens > 0 && n_heads >= 0 && n_kv_heads >= 0 && n_heads + n_kv_heads > 0 && dh > 0, "rope_store: bad sizes");
    QS_REQUIRE(n_kv_heads == 0 || (k && v && k_cache && v_cache), "rope_store: keys and values without a cache to keep them");
    QS_REQUIRE(dh % 2 == 0, "rope_store: head size %d must be even", dh);
    QS_REQUIRE(R >= 0 && R % 2 == 0 && R <= dh, "rope_store: rotary width %d must be even and within the head size %d", R, dh);
    QS_REQUIRE(page_tokens > 0 && (page_tokens & (page_tokens - 1)) == 0, "rope_store: page size %d is no power of two", page_tokens);
    int shift = 0;
    while ((1 << shift) < page_tokens) ++shift;
    const int work = (n_heads + 2 * n_kv_heads) * dh / 2;
    const int threads = work >= 2048 ? 256 : (work >= 512 ? 128 : 64);
    int per_token = 1;                       // few tokens (decode): several blocks per token
    if (T_tokens < 256) { per_token = (n_kv_heads * dh / 2 + threads - 1) / threads; if (per_token > 16) per_token = 16; if (per_token < 1) per_token = 1; }
    dim3 grid(T_tokens, per_token);
    const bool aligned = dh % 8 == 0 && dv % 8 == 0 && R % 8 == 0 && ldq % 8 == 0 && ldk % 8 == 0 && ldv % 8 == 0 &&
                         ldvf % 8 == 0 && ((uintptr_t)v_first % 16) == 0 &&
                         ((uintptr_t)q % 16) == 0 && ((uintptr_t)k % 16) == 0 && ((uintptr_t)v % 16) == 0 &&
                         ((uintptr_t)k_cache % 16) == 0 && ((uintptr_t)v_cache % 16) == 0 && ((uintptr_t)cos_sin % 16) == 0;
    if (dtype == QS_BF16 && aligned && !(half_layout && R > 0)) {
        const int work8 = (n_heads * (R / 8) + n_kv_heads * ((dh + dv) / 16));
        const int threads8 = work8 >= 512 ? 128 : 64;
        int per = 1;
        if (T_tokens < 256) { per = (n_kv_heads * ((dh + dv) / 16) + threads8 - 1) / threads8; if (per > 16) per = 16; if (per < 1) per = 1; }
        cudaError_t e = qs_launch_dependent(rope_store_vec_kernel, dim3(T_tokens, per), dim3(threads8), 0, stream,
            (__nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (size_t)ldq, (size_t)ldk, (size_t)ldv,
            n_heads, n_kv_heads, dh, R, cos_sin, max_pos, tok_slot, tok_pos, page_table, max_pages, shift,
            (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, status, settled, dv, (const __nv_bfloat16*)v_first, (size_t)ldvf, lam);
        if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "rope_store: %s", cudaGetErrorString(e));
        return qs_check_launch("rope_store");
    }
    if (dtype == QS_F32)
        qs_launch_dependent(rope_store_kernel<float>, grid, dim3(threads), 0, stream, (float*)q, (const float*)k, (const float*)v,
            (size_t)ldq, (size_t)ldk, (size_t)ldv, n_heads, n_kv_heads, dh, R, cos_sin, max_pos, tok_slot, tok_pos,
            page_table, max_pages, shift, (float*)k_cache, (float*)v_cache, status, dv, (const float*)v_first, (size_t)ldvf, lam,
            half_layout);
    else if (dtype == QS_BF16)
        qs_launch_dependent(rope_store_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, (__nv_bfloat16*)q, (const __nv_bfloat16*)k,
            (const __nv_bfloat16*)v, (size_t)ldq, (size_t)ldk, (size_t)ldv, n_heads, n_kv_heads, dh, R, cos_sin, max_pos,
            tok_slot, tok_pos, page_table, max_pages, shift, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, status, dv,
            (const __nv_bfloat16*)v_first, (size_t)ldvf, lam, half_layout);
    else return qs_fail(QS_ERR_INVALID_INPUT, "rope_store: unknown dtype %d", dtype);
    return qs_check_launch("rope_store");
}

namespace {
__device__ __forceinline__ void unpack8(const uint4 raw, float (&f)[8]) {
    const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) { f[2 * j] = __uint_as_float(u[j] << 16); f[2 * j + 1] = __uint_as_float(u[j] & 0xffff0000u); }
}

__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const __nv_bfloat162 p = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
        o[j] = *reinterpret_cast<const uint32_t*>(&p);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

// One item of a head in 16-byte pieces: src and dst point at the head's first element, w_base is the head's first
// weight.  Items below n_rot are rotated (HALF: dims [8 item, +8) paired with [R/2 + 8 item, +8); else the four
// neighbouring pairs of dims [8 item, +8)), the others are the plain dims from R on.
template <bool HALF>
__device__ __forceinline__ void norm_rot_item(const __nv_bfloat16* src, __nv_bfloat16* dst, const void* w, int w_dtype, int w_base,
                                              float rstd, int item, int n_rot, int R, const float* __restrict__ cs) {
    float a[8], wa[8];
    if (item >= n_rot) {
        const int d0 = R + 8 * (item - n_rot);
        unpack8(*reinterpret_cast<const uint4*>(src + d0), a);
        load8_as_f32(w, w_dtype, w_base + d0, wa);
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] *= rstd * wa[i];
        *reinterpret_cast<uint4*>(dst + d0) = pack8(a);
    } else if (HALF) {
        const int rp = R >> 1, d0 = 8 * item;
        float b[8], wb[8], c[16];
        unpack8(*reinterpret_cast<const uint4*>(src + d0), a);
        unpack8(*reinterpret_cast<const uint4*>(src + rp + d0), b);
        load8_as_f32(w, w_dtype, w_base + d0, wa);
        load8_as_f32(w, w_dtype, w_base + rp + d0, wb);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 x = reinterpret_cast<const float4*>(cs + 16 * item)[i];
            c[4 * i] = x.x; c[4 * i + 1] = x.y; c[4 * i + 2] = x.z; c[4 * i + 3] = x.w;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float x = a[i] * rstd * wa[i], y = b[i] * rstd * wb[i];
            a[i] = x * c[2 * i] - y * c[2 * i + 1];
            b[i] = x * c[2 * i + 1] + y * c[2 * i];
        }
        *reinterpret_cast<uint4*>(dst + d0) = pack8(a);
        *reinterpret_cast<uint4*>(dst + rp + d0) = pack8(b);
    } else {
        const int d0 = 8 * item;
        unpack8(*reinterpret_cast<const uint4*>(src + d0), a);
        load8_as_f32(w, w_dtype, w_base + d0, wa);
        const float4 c0 = reinterpret_cast<const float4*>(cs + d0)[0], c1 = reinterpret_cast<const float4*>(cs + d0)[1];
        const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float x = a[2 * i] * rstd * wa[2 * i], y = a[2 * i + 1] * rstd * wa[2 * i + 1];
            a[2 * i] = x * c[2 * i] - y * c[2 * i + 1];
            a[2 * i + 1] = x * c[2 * i + 1] + y * c[2 * i];
        }
        *reinterpret_cast<uint4*>(dst + d0) = pack8(a);
    }
}

// norm_rope_store_kernel for bfloat16 in 16-byte pieces: head sizes multiples of 8, a rotated width whose items are whole
// pieces (R a multiple of 16 by halves, of 8 by neighbours), 16-byte aligned rows.
template <bool HALF>
__global__ void norm_rope_store_vec_kernel(__nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                           const __nv_bfloat16* __restrict__ v, size_t ldq, size_t ldk, size_t ldv,
                                           const void* __restrict__ wq, int wq_dtype, const void* __restrict__ wk, int wk_dtype,
                                           float eps, int n_heads, int n_kv_heads, int dh, int dv, int R,
                                           const float* __restrict__ cos_sin, int max_pos, const int32_t* __restrict__ tok_slot,
                                           const int32_t* __restrict__ tok_pos, const int32_t* __restrict__ page_table,
                                           int max_pages, int page_shift, __nv_bfloat16* __restrict__ k_cache,
                                           __nv_bfloat16* __restrict__ v_cache, int32_t* __restrict__ status) {
    __shared__ float scratch[33];
    grid_dep_launch();
    grid_dep_wait();
    const int t = blockIdx.x, tid = threadIdx.x, stride = blockDim.x;
    const int slot = tok_slot[t];
    const int nq = n_heads * dh, nk = n_kv_heads * dh;
    __nv_bfloat16* qrow = q + (size_t)t * ldq;
    if (slot < 0) {
        for (int c = tid * 8; c < nq; c += stride * 8) *reinterpret_cast<uint4*>(qrow + c) = make_uint4(0u, 0u, 0u, 0u);
        return;
    }
    const int pos = tok_pos[t];
    if (R > 0 && (pos < 0 || pos >= max_pos)) { if (tid == 0) atomicExch(status, 1); return; }
    const float* cs = R > 0 ? cos_sin + (size_t)pos * R : nullptr;
    const __nv_bfloat16* krow = k + (size_t)t * ldk;
    float sq = 0.f, sk = 0.f, f[8];
    for (int c = tid * 8; c < nq; c += stride * 8) {
        unpack8(*reinterpret_cast<const uint4*>(qrow + c), f);
#pragma unroll
        for (int i = 0; i < 8; ++i) sq = fmaf(f[i], f[i], sq);
    }
    for (int c = tid * 8; c < nk; c += stride * 8) {
        unpack8(*reinterpret_cast<const uint4*>(krow + c), f);
#pragma unroll
        for (int i = 0; i < 8; ++i) sk = fmaf(f[i], f[i], sk);
    }
    const float rq = 1.0f / sqrtf(block_sum(sq, scratch) / (float)nq + eps);
    const float rk = nk > 0 ? 1.0f / sqrtf(block_sum(sk, scratch) / (float)nk + eps) : 0.f;
    const int n_rot = HALF ? R / 16 : R / 8, per_head = n_rot + (dh - R) / 8;
    for (int e = tid; e < n_heads * per_head; e += stride) {
        const int head = e / per_head, item = e - head * per_head;
        norm_rot_item<HALF>(qrow + head * dh, qrow + head * dh, wq, wq_dtype, head * dh, rq, item, n_rot, R, cs);
    }
    if (n_kv_heads == 0) return;
    const int page = page_table[(size_t)slot * max_pages + (pos >> page_shift)];
    if (page < 0) { if (tid == 0) atomicExch(status, 2); return; }
    const int page_tokens = 1 << page_shift;
    const size_t in_page = (size_t)(pos & (page_tokens - 1));
    for (int e = tid; e < n_kv_heads * per_head; e += stride) {
        const int kvh = e / per_head, item = e - kvh * per_head;
        norm_rot_item<HALF>(krow + kvh * dh, k_cache + (((size_t)page * n_kv_heads + kvh) * page_tokens + in_page) * dh, wk, wk_dtype,
                            kvh * dh, rk, item, n_rot, R, cs);
    }
    const int dv8 = dv / 8;
    for (int e = tid; e < n_kv_heads * dv8; e += stride) {
        const int kvh = e / dv8, c = (e - kvh * dv8) * 8;
        *reinterpret_cast<uint4*>(v_cache + (((size_t)page * n_kv_heads + kvh) * page_tokens + in_page) * dv + c) =
            *reinterpret_cast<const uint4*>(v + (size_t)t * ldv + (size_t)kvh * dv + c);
    }
}
}  // namespace

// See norm_rope_store_kernel.  wq [n_heads * dh] and wk [n_kv_heads * dh] are the two norms' weights; n_kv_heads = 0
// (k, v, the cache null): a layer that projects queries only.
QS_API int qs_norm_rope_store(void* q, const void* k, const void* v, int dtype, long long ldq, long long ldk, long long ldv,
                              const void* wq, int wq_dtype, const void* wk, int wk_dtype, float eps, int n_heads,
                              int n_kv_heads, int dh, int dv, int R, const float* cos_sin, int max_pos,
                              const int32_t* tok_slot, const int32_t* tok_pos, const int32_t* page_table, int max_pages,
                              int page_tokens, void* k_cache, void* v_cache, int T_tokens, int32_t* status, int half_layout,
                              cudaStream_t stream) {
    if (T_tokens == 0) return QS_OK;
    if (dv <= 0) dv = dh;
    QS_REQUIRE(T_tokens > 0 && n_heads > 0 && n_kv_heads >= 0 && dh > 0 && q && wq, "norm_rope_store: bad sizes");
    QS_REQUIRE(n_kv_heads == 0 || (k && v && wk && k_cache && v_cache && page_table), "norm_rope_store: keys without their norm or cache");
    QS_REQUIRE(dh % 2 == 0, "norm_rope_store: head size %d must be even", dh);
    QS_REQUIRE(R >= 0 && R % 2 == 0 && R <= dh, "norm_rope_store: rotary width %d must be even and within the head size %d", R, dh);
    QS_REQUIRE(page_tokens > 0 && (page_tokens & (page_tokens - 1)) == 0, "norm_rope_store: page size %d is no power of two", page_tokens);
    int shift = 0;
    while ((1 << shift) < page_tokens) ++shift;
    const int work = n_heads * dh;
    const int threads = work >= 2048 ? 256 : 128;
    cudaError_t e;
    const bool rot_fits = R == 0 || (cos_sin && ((uintptr_t)cos_sin % 16) == 0 && (half_layout ? R % 16 == 0 : R % 8 == 0));
    const bool aligned = dtype == QS_BF16 && dh % 8 == 0 && dv % 8 == 0 && rot_fits && ldq % 8 == 0 && ldk % 8 == 0 && ldv % 8 == 0 &&
                         ((uintptr_t)q % 16) == 0 && ((uintptr_t)k % 16) == 0 && ((uintptr_t)v % 16) == 0 &&
                         ((uintptr_t)k_cache % 16) == 0 && ((uintptr_t)v_cache % 16) == 0 && ((uintptr_t)wq % 32) == 0 && ((uintptr_t)wk % 32) == 0;
    if (aligned) {
        typedef __nv_bfloat16 bf16;
        const int threads8 = work >= 8192 ? 256 : (work >= 2048 ? 128 : 64);
#define GOV(HALF) e = qs_launch_dependent(norm_rope_store_vec_kernel<HALF>, dim3(T_tokens), dim3(threads8), 0, stream, (bf16*)q, (const bf16*)k, \
        (const bf16*)v, (size_t)ldq, (size_t)ldk, (size_t)ldv, wq, wq_dtype, wk, wk_dtype, eps, n_heads, n_kv_heads, dh, dv, cos_sin ? R : 0, \
        cos_sin, max_pos, tok_slot, tok_pos, page_table, max_pages, shift, (bf16*)k_cache, (bf16*)v_cache, status)
        if (half_layout) GOV(true); else GOV(false);
#undef GOV
        if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "norm_rope_store: %s", cudaGetErrorString(e));
        return qs_check_launch("norm_rope_store");
    }
#define GO(T) e = qs_launch_dependent(norm_rope_store_kernel<T>, dim3(T_tokens), dim3(threads), 0, stream, (T*)q, (const T*)k, (const T*)v, \
        (size_t)ldq, (size_t)ldk, (size_t)ldv, wq, wq_dtype, wk, wk_dtype, eps, n_heads, n_kv_heads, dh, dv, R, cos_sin, max_pos, \
        tok_slot, tok_pos, page_table, max_pages, shift, (T*)k_cache, (T*)v_cache, status, half_layout)
    if (dtype == QS_F32) GO(float);
    else if (dtype == QS_BF16) GO(__nv_bfloat16);
    else return qs_fail(QS_ERR_INVALID_INPUT, "norm_rope_store: unknown dtype %d", dtype);
#undef GO
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "norm_rope_store: %s", cudaGetErrorString(e));
    return qs_check_launch("norm_rope_store");
}

QS_API int qs_attention(void* out, const void* q, int dtype, long long ldo, long long ldq,
                        const void* k_cache, const void* v_cache,
                        const int32_t* page_table, int max_pages, int page_tokens,
                        const int32_t* tok_slot, const int32_t* tok_pos, int T_tokens,
                        int n_heads, int n_kv_heads, int dh, float scale, int window,
                        int32_t* status, int dv, float softcap, int chunk, int keep_first, const float* sink,
                        int maps, int out_dtype, cudaStream_t stream) {
    if (T_tokens == 0) return QS_OK;
    if (dv <= 0) dv = dh;
    if (maps <= 0) maps = 1;
    if (out_dtype < 0) out_dtype = dtype;
    QS_REQUIRE(out_dtype == dtype || out_dtype == QS_F32, "attention: a result of type %d from queries of type %d", out_dtype, dtype);
    QS_REQUIRE(dv <= 512, "attention: value head size %d above 512", dv);
    QS_REQUIRE(T_tokens > 0 && n_heads > 0 && n_kv_heads > 0 && dh > 0, "attention: bad sizes");
    QS_REQUIRE(chunk >= 0 && keep_first >= 0 && !(chunk > 0 && window > 0), "attention: a window of %d and chunks of %d", window, chunk);
    QS_REQUIRE(n_heads % maps == 0 && (n_heads / maps) % n_kv_heads == 0, "attention: %d query heads in %d maps over %d key heads",
               n_heads, maps, n_kv_heads);
    QS_REQUIRE(n_heads % n_kv_heads == 0, "attention: %d query heads are no multiple of %d key heads", n_heads, n_kv_heads);
    QS_REQUIRE(dh <= 2048, "attention: head size %d above 2048", dh);      // a warp's query in shared memory: 4 warps x dh floats
    QS_REQUIRE(page_tokens > 0 && (page_tokens & (page_tokens - 1)) == 0, "attention: page size %d is no power of two", page_tokens);
    QS_REQUIRE(window >= 0, "attention: negative window");
    int shift = 0;
    while ((1 << shift) < page_tokens) ++shift;
    if (dtype == QS_F32)
        return launch_attention<float, float>(out, q, ldo, ldq, k_cache, v_cache, page_table, max_pages, shift, tok_slot,
                                       tok_pos, T_tokens, n_heads, n_kv_heads, dh, scale, window, status, dv, softcap,
                                       chunk, keep_first, sink, maps, stream);
    if (dtype == QS_BF16 && out_dtype == QS_F32)
        return launch_attention<__nv_bfloat16, float>(out, q, ldo, ldq, k_cache, v_cache, page_table, max_pages, shift,
                                                      tok_slot, tok_pos, T_tokens, n_heads, n_kv_heads, dh, scale, window,
                                                      status, dv, softcap, chunk, keep_first, sink, maps, stream);
    if (dtype == QS_BF16)
        return launch_attention<__nv_bfloat16, __nv_bfloat16>(out, q, ldo, ldq, k_cache, v_cache, page_table, max_pages, shift,
                                                              tok_slot, tok_pos, T_tokens, n_heads, n_kv_heads, dh, scale, window,
                                                              status, dv, softcap, chunk, keep_first, sink, maps, stream);
    return qs_fail(QS_ERR_INVALID_INPUT, "attention: unknown dtype %d", dtype);
}

// Two attention maps over the same values, joined: for every head, o = a1 - lam * a2, divided by its root mean
// square over the head's dv values (eps inside the root), times `mult`.  a [rows, heads * 2 * dv], per head
// [map 1 | map 2]; out [rows, heads * dv].  One warp per (row, head); 32-bit throughout, rounded once.
namespace {
template <typename TI, typename TO>
__global__ void pair_diff_norm_kernel(TO* __restrict__ out, size_t ldo, const TI* __restrict__ a, size_t lda, int rows,
                                      int heads, int dv, float lam, float mult, float eps) {
    grid_dep_launch();
    grid_dep_wait();
    const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * warps + (threadIdx.x >> 5);
    if (item >= (long long)rows * heads) return;
    const int r = (int)(item / heads), hd = (int)(item % heads);
    const TI* a1 = a + (size_t)r * lda + (size_t)hd * 2 * dv;
    const TI* a2 = a1 + dv;
    float sq = 0.f;
    for (int i = lane; i < dv; i += 32) { const float o = fmaf(-lam, to_f32(a2[i]), to_f32(a1[i])); sq = fmaf(o, o, sq); }
    sq = warp_sum(sq);
    const float f = mult / sqrtf(sq / (float)dv + eps);
    TO* dst = out + (size_t)r * ldo + (size_t)hd * dv;
    for (int i = lane; i < dv; i += 32) dst[i] = from_f32<TO>(fmaf(-lam, to_f32(a2[i]), to_f32(a1[i])) * f);
}
}  // namespace

QS_API int qs_pair_diff_norm(void* out, int out_dtype, long long ldo, const void* a, int a_dtype, long long lda, int rows,
                             int heads, int dv, float lam, float mult, float eps, cudaStream_t stream) {
    if (rows == 0) return QS_OK;
    QS_REQUIRE(rows > 0 && heads > 0 && dv > 0, "pair_diff_norm: bad sizes");
    typedef __nv_bfloat16 bf16;
    const int warps = 4;
    const int blocks = (int)(((long long)rows * heads + warps - 1) / warps);
    cudaError_t e;
#define GO(TI, TO) e = qs_launch_dependent(pair_diff_norm_kernel<TI, TO>, dim3(blocks), dim3(warps * 32), 0, stream, (TO*)out, \
                                           (size_t)ldo, (const TI*)a, (size_t)lda, rows, heads, dv, lam, mult, eps)
    if (a_dtype == QS_F32 && out_dtype == QS_F32) GO(float, float);
    else if (a_dtype == QS_F32 && out_dtype == QS_BF16) GO(float, bf16);
    else if (a_dtype == QS_BF16 && out_dtype == QS_BF16) GO(bf16, bf16);
    else return qs_fail(QS_ERR_INVALID_INPUT, "pair_diff_norm: unsupported types a=%d out=%d", a_dtype, out_dtype);
#undef GO
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "pair_diff_norm: %s", cudaGetErrorString(e));
    return qs_check_launch("pair_diff_norm");
}
