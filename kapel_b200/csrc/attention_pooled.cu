// Attention over a sliding window plus pooled blocks, with the heads' weights mixed after the softmax.
//
//  proj_rope_append   one block a row of the stacked q|k|v product (a tensor or split-K partial sums):
//                     biases, an RMS norm over the whole query projection and over the whole key
//                     projection, the rotation of the first `rotary` components of every head (pairs
//                     (i, i + rotary/2) or neighbours (2i, 2i+1)), the values mixed with another
//                     layer's values of the same rows (v <- (1 - l) v + l v_other), queries written
//                     out, keys and values to the paged cache at the row's line.
//  pool_blocks        a row whose position ends a block of `pool` positions reads the block's keys and
//                     values back from the cache (as the cache holds them), and leaves their means in
//                     the request's slot of a 32-bit table [slots, blocks, kv_heads, d + dv].
//  pooled_attention   a query that has seen c positions reads the tokens [max(0, c - window), c) and
//                     the blocks b < floor((c - window) / pool) (those that lie wholly below the
//                     window); one softmax over both; the heads' weights are mixed
//                     (w'_h = sum_g talk[h, g] w_g) before they meet the values of h's kv head.
//                     score = q.k * scale * temp[h].
//
// The mix needs every head's normalised weight of a key, so a row's heads run in one block, in two
// walks over the keys: the first leaves each head's maximum and sum, the second computes the weights
// again, normalises, mixes and adds the values up. With few rows the keys are cut into slices across
// blocks: slice statistics, then slice sums (already normalised, so they simply add up), then their
// sum in slice order. Scores, softmax, the mix and all sums are 32-bit.
#include "common.cuh"

namespace kb {

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float pooled_exp(float x) { return __expf(x); }
template <> __device__ __forceinline__ float pooled_exp<float>(float x) { return expf(x); }

// Eight neighbours of a row that starts on a 16-byte boundary, as 32-bit values.
__device__ __forceinline__ void pooled_load8(const float* p, float (&x)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}
__device__ __forceinline__ void pooled_load8(const bf16* p, float (&x)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        x[2 * i] = f.x;
        x[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ float pooled_dot8(const float (&k)[8], const float* q, float acc) {
    const float4 a = *reinterpret_cast<const float4*>(q), b = *reinterpret_cast<const float4*>(q + 4);
    acc = fmaf(k[0], a.x, acc); acc = fmaf(k[1], a.y, acc); acc = fmaf(k[2], a.z, acc); acc = fmaf(k[3], a.w, acc);
    acc = fmaf(k[4], b.x, acc); acc = fmaf(k[5], b.y, acc); acc = fmaf(k[6], b.z, acc); acc = fmaf(k[7], b.w, acc);
    return acc;
}

// ------------------------------------------------------------------------------ proj_rope_append
template <typename TS, typename TW, typename TO>
__global__ void proj_rope_append_kernel(const Src<TS> src, int row_width, int q_off, int k_off, int v_off,
                                        const TW* __restrict__ bq, const TW* __restrict__ bk, const TW* __restrict__ bv,
                                        const TW* __restrict__ wq, float eps_q, float off_q,
                                        const TW* __restrict__ wk, float eps_k, float off_k,
                                        const float2* __restrict__ cos_sin, int rotary, int neighbours,
                                        const float* __restrict__ v_other, const TW* __restrict__ lambda,
                                        float* __restrict__ v_keep,
                                        const int* __restrict__ lines, TO* __restrict__ q_out, TO* __restrict__ k_table,
                                        TO* __restrict__ v_table, int hq, int hkv, int d, int dv, long long table_lines,
                                        int page_size) {
    extern __shared__ float row[];                          // q [hq d] | k [hkv d]
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const size_t base = (size_t)r * row_width;
    const int nq = hq * d, nk = hkv * d, nv = hkv * dv;
    float* sq = row;
    float* sk = row + nq;
    float ssq = 0.f, ssk = 0.f;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) {
        float v = src.at(base + q_off + i);
        if (bq != nullptr) v += Elem<TW>::load(bq + i);
        sq[i] = v;
        ssq = fmaf(v, v, ssq);
    }
    for (int i = threadIdx.x; i < nk; i += blockDim.x) {
        float v = src.at(base + k_off + i);
        if (bk != nullptr) v += Elem<TW>::load(bk + i);
        sk[i] = v;
        ssk = fmaf(v, v, ssk);
    }
    if (wq != nullptr) {
        ssq = block_sum(ssq, scratch);
        const float inv = 1.f / sqrtf(ssq / (float)nq + eps_q);
        for (int i = threadIdx.x; i < nq; i += blockDim.x) sq[i] = sq[i] * inv * (off_q + Elem<TW>::load(wq + i));
    }
    if (wk != nullptr) {
        ssk = block_sum(ssk, scratch);
        const float inv = 1.f / sqrtf(ssk / (float)nk + eps_k);
        for (int i = threadIdx.x; i < nk; i += blockDim.x) sk[i] = sk[i] * inv * (off_k + Elem<TW>::load(wk + i));
    }
    __syncthreads();
    const int half = rotary >> 1;
    if (half > 0) {
        for (int u = threadIdx.x; u < (hq + hkv) * half; u += blockDim.x) {
            const int h = u / half, i = u - h * half;
            float* x = row + (size_t)h * d;                 // the heads of q and then of k lie d apart
            const int ia = neighbours ? 2 * i : i, ib = neighbours ? 2 * i + 1 : i + half;
            float a = x[ia], b = x[ib];
            rope_rotate(a, b, cos_sin[(size_t)r * half + i]);
            x[ia] = a;
            x[ib] = b;
        }
        __syncthreads();
    }
    for (int i = threadIdx.x; i < nq; i += blockDim.x) Elem<TO>::store(q_out + (size_t)r * nq + i, sq[i]);
    long long line = -1;
    if (k_table != nullptr) {
        line = lines[r];
        if (line >= table_lines) line = -1;
    }
    if (line >= 0)
        for (int i = threadIdx.x; i < nk; i += blockDim.x) {
            const int h = i / d, c = i - h * d;
            Elem<TO>::store(k_table + kv_row(line, h, hkv, page_size) * d + c, sk[i]);
        }
    const float lam = lambda != nullptr ? Elem<TW>::load(lambda) : 0.f;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
        float v = src.at(base + v_off + i);
        if (bv != nullptr) v += Elem<TW>::load(bv + i);
        if (v_keep != nullptr) v_keep[(size_t)r * nv + i] = v;
        if (v_other != nullptr) v = (1.f - lam) * v + lam * v_other[(size_t)r * nv + i];
        if (line >= 0) {
            const int h = i / dv, c = i - h * dv;
            Elem<TO>::store(v_table + kv_row(line, h, hkv, page_size) * dv + c, v);
        }
    }
}

// ----------------------------------------------------------------------------------- pool_blocks
template <typename T>
__global__ void pool_blocks_kernel(const T* __restrict__ k_table, const T* __restrict__ v_table,
                                   const int* __restrict__ block_table, int table_width, int n_pages,
                                   const int* __restrict__ row_entry, const int* __restrict__ positions,
                                   const int* __restrict__ lines, const int* __restrict__ slots, float* __restrict__ pooled,
                                   long long slot_stride, int n_slots, int max_blocks, int pool, int hkv, int d, int dv,
                                   int page_size) {
    const int r = blockIdx.x;
    if (lines[r] < 0) return;                               // a row of no token
    const int pos = positions[r];
    if ((pos + 1) % pool != 0) return;                      // the row does not end a block
    const int b = pos / pool;
    const int entry = row_entry[r];
    const int slot = slots[entry];
    if (b >= max_blocks || slot <= 0 || slot >= n_slots) return;
    const int wide = d + dv;
    float* out = pooled + (size_t)slot * slot_stride + (size_t)b * hkv * wide;
    for (int i = threadIdx.x; i < hkv * wide; i += blockDim.x) {
        const int g = i / wide, c = i - g * wide;
        float acc = 0.f;
        for (int t = 0; t < pool; ++t) {
            const int p = b * pool + t;
            const int lp = p / page_size;
            const int page = lp < table_width ? block_table[(size_t)entry * table_width + lp] : -1;
            if (page < 0 || page >= n_pages) continue;      // a fault of the cache manager; never with a window >= pool
            const long long line = (long long)page * page_size + p % page_size;
            const size_t at = kv_row(line, g, hkv, page_size);
            acc += c < d ? Elem<T>::load(k_table + at * d + c) : Elem<T>::load(v_table + at * dv + (c - d));
        }
        out[i] = acc / (float)pool;
    }
}

// ------------------------------------------------------------------------------ pooled_attention
constexpr int PA_THREADS = 256;
constexpr int PA_WARPS = PA_THREADS / 32;
constexpr int PA_CHUNK = 64;          // keys a step
constexpr int PA_LPK = 8;             // lanes that share a (key, head) dot product

struct PooledParams {
    const void* q;             // [rows, hq, d]
    const void* k_table;       // [pages, hkv, page_size, d]
    const void* v_table;       // [pages, hkv, page_size, dv]
    const float* pooled;       // [slots, max_blocks, hkv, d + dv]
    const int* block_table;    // [entries, table_width]
    const int* row_entry;      // [rows]
    const int* row_count;      // [rows]
    const int* slots;          // [entries]
    const float* talk;         // [hq, hq] or null (no mix)
    const float* temp;         // [hq] or null
    void* out;                 // [rows, hq, dv]
    float* stats;              // [rows, splits, hq, 2] (with splits > 1)
    float* partial;            // [rows, splits, hq, dv] (with splits > 1)
    float* kept_scores;        // [rows, splits, hq, split_keys] (with splits > 1): the first walk's scores, which the second reads back
    long long slot_stride;
    int rows, hq, hkv, d, dv, page_size, table_width, n_pages, n_slots, max_blocks;
    int window, pool;          // window 0: every token is seen and no block; pool 0: no blocks
    int splits, split_keys;    // keys a slice (a multiple of PA_CHUNK)
    int mode;                  // 0: all in one; 1: a slice's statistics; 2: a slice's sums
    float scale;
};

// What a row that has seen `count` positions reads: `nb` blocks, then the tokens from `first`.
__device__ __forceinline__ void pooled_extent(const PooledParams& p, int count, int& nb, int& first) {
    first = (p.window > 0 && count > p.window) ? count - p.window : 0;
    nb = (p.pool > 0 && p.window > 0 && count > p.window) ? min((count - p.window) / p.pool, p.max_blocks) : 0;
}

// OPT: value components a thread adds up (hq * dv <= PA_THREADS * OPT).
template <typename T, int OPT>
__global__ void __launch_bounds__(PA_THREADS)
pooled_attention_kernel(const PooledParams p) {
    extern __shared__ __align__(16) float smem[];
    const int hq = p.hq, d = p.d, dv = p.dv, group = p.hq / p.hkv;
    float* sq = smem;                                   // [hq][d]
    float* ss = sq + (size_t)hq * d;                    // [hq][CHUNK] scores, then normalised weights
    float* pm = ss + (size_t)hq * PA_CHUNK;             // [hq][CHUNK] mixed weights
    float* stalk = pm + (size_t)hq * PA_CHUNK;          // [hq][hq]
    float* sm = stalk + (size_t)hq * hq;                // [hq] maxima
    float* sz = sm + hq;                                // [hq] sums
    long long* skey = reinterpret_cast<long long*>((reinterpret_cast<uintptr_t>(sz + hq) + 7) & ~(uintptr_t)7);   // [CHUNK] a token's row of kv head 0 in the tables, or -1 - block
    const int r = blockIdx.x, z = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int count = p.row_count[r];
    T* out = static_cast<T*>(p.out);
    int nb, first;
    pooled_extent(p, max(count, 0), nb, first);
    const int n_keys = count > 0 ? nb + (count - first) : 0;
    const int j_lo = p.mode == 0 ? 0 : z * p.split_keys;
    const int j_hi = p.mode == 0 ? n_keys : min(n_keys, (z + 1) * p.split_keys);
    if (n_keys <= 0) {
        if (p.mode == 0)
            for (int i = tid; i < hq * dv; i += PA_THREADS) Elem<T>::store(out + (size_t)r * hq * dv + i, 0.f);
        // with slices: statistics of -inf / 0 and sums of 0, so that the last kernel writes zeros
    }
    const int entry = p.row_entry[r];
    const int slot = p.slots[entry];
    const float* pooled = p.pooled + (size_t)((slot > 0 && slot < p.n_slots) ? slot : 0) * p.slot_stride;
    const T* q = static_cast<const T*>(p.q) + (size_t)r * hq * d;
    for (int i = tid; i < hq * d; i += PA_THREADS) sq[i] = Elem<T>::load(q + i);
    for (int i = tid; i < hq * hq; i += PA_THREADS) stalk[i] = p.talk != nullptr ? p.talk[i] : ((i / hq) == (i % hq) ? 1.f : 0.f);
    if (tid < hq) { sm[tid] = -INFINITY; sz[tid] = 0.f; }
    __syncthreads();
    const T* kt = static_cast<const T*>(p.k_table);
    const T* vt = static_cast<const T*>(p.v_table);
    const int wide = d + dv;

    const bool vec = d % 8 == 0;                        // rows of keys start on 16-byte boundaries
    const bool vec_means = vec && wide % 4 == 0;
    // where the keys [j0, j0 + n) lie, into skey
    auto keys_at = [&](int j0, int n) {
        for (int j = tid; j < n; j += PA_THREADS) {
            const int key = j0 + j;
            long long at;
            if (key < nb) {
                at = -1 - (long long)key;
            } else {
                const int pos = first + (key - nb);
                const int lp = pos / p.page_size;
                const int page = lp < p.table_width ? p.block_table[(size_t)entry * p.table_width + lp] : -1;
                // the token's row of kv head 0 in the tables [pages, kv heads, page size, .]: head g's lies g pages' lines further
                at = (page >= 0 && page < p.n_pages) ? ((long long)page * p.hkv) * p.page_size + pos % p.page_size : (long long)0x7fffffffffffffffll;
            }
            skey[j] = at;
        }
        __syncthreads();
    };
    // the scores of the keys [j0, j0 + n) into ss
    auto scores = [&](int j0, int n) {
        keys_at(j0, n);
        const int sub = tid / PA_LPK, li = tid % PA_LPK;
        const unsigned mates = ((1u << PA_LPK) - 1u) << (lane & ~(PA_LPK - 1));    // the lanes of this dot product: groups leave the loop at different times
        for (int item = sub; item < n * hq; item += PA_THREADS / PA_LPK) {
            const int j = item / hq, h = item - j * hq;
            const int g = h / group;
            const long long at = skey[j];
            float dot = 0.f;
            const float* qh = sq + (size_t)h * d;
            if (at == 0x7fffffffffffffffll) {
                dot = 0.f;
            } else if (at < 0) {
                const float* kp = pooled + ((size_t)(-1 - at) * p.hkv + g) * wide;
                if (vec_means) {
                    for (int c = li * 8; c < d; c += PA_LPK * 8) {
                        float kx[8];
                        pooled_load8(kp + c, kx);
                        dot = pooled_dot8(kx, qh + c, dot);
                    }
                } else {
                    for (int c = li; c < d; c += PA_LPK) dot = fmaf(kp[c], qh[c], dot);
                }
            } else {
                const T* kp = kt + (size_t)(at + (long long)g * p.page_size) * d;
                if (vec) {
                    for (int c = li * 8; c < d; c += PA_LPK * 8) {
                        float kx[8];
                        pooled_load8(kp + c, kx);
                        dot = pooled_dot8(kx, qh + c, dot);
                    }
                } else {
                    for (int c = li; c < d; c += PA_LPK) dot = fmaf(Elem<T>::load(kp + c), qh[c], dot);
                }
            }
#pragma unroll
            for (int o = PA_LPK / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(mates, dot, o);
            if (li == 0) {
                float s = dot * p.scale;
                if (p.temp != nullptr) s *= p.temp[h];
                ss[h * PA_CHUNK + j] = at == 0x7fffffffffffffffll ? -INFINITY : s;
            }
        }
        __syncthreads();
    };

    // ---- the first walk: every head's maximum and sum over the keys of this block
    if (p.mode != 2) {
        for (int j0 = j_lo; j0 < j_hi; j0 += PA_CHUNK) {
            const int n = min(PA_CHUNK, j_hi - j0);
            scores(j0, n);
            for (int h = warp; h < hq; h += PA_WARPS) {
                float mx = -INFINITY;
                for (int j = lane; j < n; j += 32) mx = fmaxf(mx, ss[h * PA_CHUNK + j]);
                mx = warp_max(mx);
                const float old = sm[h];
                const float top = fmaxf(old, mx);
                float l = 0.f;
                if (top != -INFINITY)
                    for (int j = lane; j < n; j += 32) l += pooled_exp<T>(ss[h * PA_CHUNK + j] - top);
                l = warp_sum(l);
                if (lane == 0) {
                    sz[h] = (old == -INFINITY ? 0.f : sz[h] * pooled_exp<T>(old - top)) + l;
                    sm[h] = top;
                }
            }
            if (p.mode == 1) {
                float* keep = p.kept_scores + ((size_t)r * p.splits + z) * hq * p.split_keys + (j0 - j_lo);
                for (int i = tid; i < hq * n; i += PA_THREADS) {
                    const int h = i / n, j = i - h * n;
                    keep[(size_t)h * p.split_keys + j] = ss[h * PA_CHUNK + j];
                }
            }
            __syncthreads();
        }
        if (p.mode == 1) {
            if (tid < hq) {
                float* st = p.stats + (((size_t)r * p.splits + z) * hq + tid) * 2;
                st[0] = sm[tid];
                st[1] = sz[tid];
            }
            return;
        }
    } else {
        // the slices' statistics merged in slice order
        if (tid < hq) {
            float top = -INFINITY;
            for (int s = 0; s < p.splits; ++s) top = fmaxf(top, p.stats[(((size_t)r * p.splits + s) * hq + tid) * 2]);
            float total = 0.f;
            for (int s = 0; s < p.splits; ++s) {
                const float* st = p.stats + (((size_t)r * p.splits + s) * hq + tid) * 2;
                if (st[0] != -INFINITY) total += st[1] * pooled_exp<T>(st[0] - top);
            }
            sm[tid] = top;
            sz[tid] = total;
        }
        __syncthreads();
    }

    // ---- the second walk: weights, normalised, mixed, times the values
    constexpr int ACC = OPT < 8 ? 8 : OPT;              // (eight neighbours a thread where the values' rows allow 16-byte loads)
    const bool vec_values = dv % 8 == 0 && d % 4 == 0;
    float acc[ACC];
#pragma unroll
    for (int u = 0; u < ACC; ++u) acc[u] = 0.f;
    for (int j0 = j_lo; j0 < j_hi; j0 += PA_CHUNK) {
        const int n = min(PA_CHUNK, j_hi - j0);
        if (p.mode == 2) {
            keys_at(j0, n);
            const float* keep = p.kept_scores + ((size_t)r * p.splits + z) * hq * p.split_keys + (j0 - j_lo);
            for (int i = tid; i < hq * n; i += PA_THREADS) {
                const int h = i / n, j = i - h * n;
                ss[h * PA_CHUNK + j] = keep[(size_t)h * p.split_keys + j];
            }
            __syncthreads();
        } else {
            scores(j0, n);
        }
        for (int i = tid; i < hq * n; i += PA_THREADS) {
            const int h = i / n, j = i - h * n;
            const float s = ss[h * PA_CHUNK + j];
            ss[h * PA_CHUNK + j] = (s == -INFINITY || sz[h] <= 0.f) ? 0.f : pooled_exp<T>(s - sm[h]) / sz[h];
        }
        __syncthreads();
        for (int i = tid; i < hq * n; i += PA_THREADS) {
            const int h = i / n, j = i - h * n;
            float w = 0.f;
            for (int g = 0; g < hq; ++g) w = fmaf(stalk[h * hq + g], ss[g * PA_CHUNK + j], w);
            pm[h * PA_CHUNK + j] = w;
        }
        __syncthreads();
        if (vec_values) {
#pragma unroll
            for (int u8 = 0; u8 < ACC / 8; ++u8) {
                const int o = (tid + u8 * PA_THREADS) * 8;
                if (o >= hq * dv) break;
                const int h = o / dv, c = o - h * dv;
                const int g = h / group;
                for (int j = 0; j < n; ++j) {
                    const long long at = skey[j];
                    if (at == 0x7fffffffffffffffll) continue;
                    float vx[8];
                    if (at < 0) pooled_load8(pooled + ((size_t)(-1 - at) * p.hkv + g) * wide + d + c, vx);
                    else pooled_load8(vt + (size_t)(at + (long long)g * p.page_size) * dv + c, vx);
                    const float w = pm[h * PA_CHUNK + j];
#pragma unroll
                    for (int k = 0; k < 8; ++k) acc[u8 * 8 + k] = fmaf(w, vx[k], acc[u8 * 8 + k]);
                }
            }
        } else
#pragma unroll
        for (int u = 0; u < OPT; ++u) {
            const int o = tid + u * PA_THREADS;
            if (o >= hq * dv) break;
            const int h = o / dv, c = o - h * dv;
            const int g = h / group;
            float a = acc[u];
            for (int j = 0; j < n; ++j) {
                const long long at = skey[j];
                if (at == 0x7fffffffffffffffll) continue;
                const float v = at < 0 ? pooled[((size_t)(-1 - at) * p.hkv + g) * wide + d + c]
                                       : Elem<T>::load(vt + (size_t)(at + (long long)g * p.page_size) * dv + c);
                a = fmaf(pm[h * PA_CHUNK + j], v, a);
            }
            acc[u] = a;
        }
        __syncthreads();
    }
    if (n_keys <= 0 && p.mode == 0) return;                 // zeros were written above
    if (vec_values) {
#pragma unroll
        for (int u = 0; u < ACC; ++u) {
            const int o = (tid + (u >> 3) * PA_THREADS) * 8 + (u & 7);
            if (o >= hq * dv) break;
            if (p.mode == 0) Elem<T>::store(out + (size_t)r * hq * dv + o, acc[u]);
            else p.partial[((size_t)r * p.splits + z) * hq * dv + o] = acc[u];
        }
        return;
    }
#pragma unroll
    for (int u = 0; u < OPT; ++u) {
        const int o = tid + u * PA_THREADS;
        if (o >= hq * dv) break;
        if (p.mode == 0) Elem<T>::store(out + (size_t)r * hq * dv + o, acc[u]);
        else p.partial[((size_t)r * p.splits + z) * hq * dv + o] = acc[u];
    }
}

template <typename T>
__global__ void pooled_sum_kernel(T* __restrict__ out, const float* __restrict__ partial, long long rows, int splits, int width) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * width) return;
    const long long r = i / width;
    const int c = (int)(i - r * width);
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) acc += partial[((size_t)r * splits + s) * width + c];
    Elem<T>::store(out + i, acc);
}

static size_t pooled_smem_bytes(int hq, int d) {
    return ((size_t)hq * d + 2 * (size_t)hq * PA_CHUNK + (size_t)hq * hq + 2 * hq + 2) * sizeof(float) + PA_CHUNK * sizeof(long long);
}

template <typename T, int OPT>
static int launch_pooled(const PooledParams& p, cudaStream_t s) {
    const size_t smem = pooled_smem_bytes(p.hq, p.d);
    if (smem > 48 * 1024) {
        if (smem > 200 * 1024) return fail("pooled_attention: %d heads of %d need %zu bytes of shared memory", p.hq, p.d, smem);
        cudaFuncSetAttribute(pooled_attention_kernel<T, OPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
    dim3 grid(p.rows, p.mode == 0 ? 1 : p.splits);
    pooled_attention_kernel<T, OPT><<<grid, PA_THREADS, smem, s>>>(p);
    return check_launch("pooled_attention");
}

template <typename T>
static int dispatch_pooled(const PooledParams& p, cudaStream_t s) {
    const int outs = p.hq * p.dv;
    if (outs <= PA_THREADS * 4) return launch_pooled<T, 4>(p, s);
    if (outs <= PA_THREADS * 16) return launch_pooled<T, 16>(p, s);
    if (outs <= PA_THREADS * 64) return launch_pooled<T, 64>(p, s);
    return fail("pooled_attention: %d heads of %d value components are more than %d", p.hq, p.dv, PA_THREADS * 64);
}

template <typename T>
static int run_pooled(PooledParams p, cudaStream_t s) {
    if (p.splits <= 1) {
        p.mode = 0;
        return dispatch_pooled<T>(p, s);
    }
    p.mode = 1;
    if (int e = dispatch_pooled<T>(p, s)) return e;
    p.mode = 2;
    if (int e = dispatch_pooled<T>(p, s)) return e;
    const long long n = (long long)p.rows * p.hq * p.dv;
    pooled_sum_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, s>>>(static_cast<T*>(p.out), p.partial, p.rows, p.splits, p.hq * p.dv);
    return check_launch("pooled_attention sum");
}

}  // namespace kb

using namespace kb;

extern "C" int kb_pooled_attention_chunk() { return PA_CHUNK; }

extern "C" int kb_proj_rope_append(const void* src, int src_dt, int splits, long long split_stride, int row_width, int q_off,
                                   int k_off, int v_off, const void* bq, const void* bk, const void* bv, const void* wq, float eps_q,
                                   float off_q, const void* wk, float eps_k, float off_k, int w_dt, const float* cos_sin, int rotary,
                                   int neighbours, const float* v_other, const void* lambda, float* v_keep, const int* lines,
                                   void* q_out, void* k_table, void* v_table, int out_dt, int rows, int hq, int hkv, int d, int dv,
                                   int write_kv, long long table_lines, int page_size, void* stream) {
    KB_REQUIRE(rows >= 0 && hq > 0 && hkv > 0 && d > 0 && dv > 0, "proj_rope_append: rows %d, heads %d / %d, sizes %d / %d", rows, hq, hkv, d, dv);
    KB_REQUIRE(splits >= 1 && row_width > 0, "proj_rope_append: %d slices of rows of %d", splits, row_width);
    KB_REQUIRE(q_off >= 0 && k_off >= 0 && v_off >= 0 && q_off + hq * d <= row_width && k_off + hkv * d <= row_width && v_off + hkv * dv <= row_width,
               "proj_rope_append: offsets %d, %d, %d do not fit rows of %d", q_off, k_off, v_off, row_width);
    KB_REQUIRE(rotary >= 0 && rotary % 2 == 0 && rotary <= d, "proj_rope_append: %d rotated components of %d", rotary, d);
    KB_REQUIRE(rotary == 0 || cos_sin != nullptr, "proj_rope_append: a rotation without its table");
    KB_REQUIRE((v_other == nullptr) == (lambda == nullptr), "proj_rope_append: other values and their weight come together");
    KB_REQUIRE(!write_kv || (lines != nullptr && k_table != nullptr && v_table != nullptr && page_size > 0), "proj_rope_append: a cache write without its tables");
    if (rows == 0) return 0;
    const size_t smem = (size_t)(hq + hkv) * d * sizeof(float);
    KB_REQUIRE(smem <= 200 * 1024, "proj_rope_append: rows of %d query and key components do not fit shared memory", (hq + hkv) * d);
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = (hq + hkv) * d >= 2048 ? 512 : 256;
#define KB_PRA(TS, TW, TO)                                                                                                      \
    do {                                                                                                                        \
        if (smem > 48 * 1024) cudaFuncSetAttribute(proj_rope_append_kernel<TS, TW, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        proj_rope_append_kernel<TS, TW, TO><<<rows, threads, smem, s>>>(                                                        \
            Src<TS>{(const TS*)src, splits, (size_t)split_stride}, row_width, q_off, k_off, v_off, (const TW*)bq, (const TW*)bk,   \
            (const TW*)bv, (const TW*)wq, eps_q, off_q, (const TW*)wk, eps_k, off_k, (const float2*)cos_sin, rotary, neighbours, \
            v_other, (const TW*)lambda, v_keep, lines, (TO*)q_out, write_kv ? (TO*)k_table : nullptr, write_kv ? (TO*)v_table : nullptr, \
            hq, hkv, d, dv, table_lines, page_size);                                                                            \
    } while (0)
    if (src_dt == KB_DT_F32 && w_dt == KB_DT_F32 && out_dt == KB_DT_F32) KB_PRA(float, float, float);
    else if (src_dt == KB_DT_F32 && w_dt == KB_DT_BF16 && out_dt == KB_DT_BF16) KB_PRA(float, bf16, bf16);
    else if (src_dt == KB_DT_BF16 && w_dt == KB_DT_BF16 && out_dt == KB_DT_BF16) KB_PRA(bf16, bf16, bf16);
    else if (src_dt == KB_DT_F32 && w_dt == KB_DT_F32 && out_dt == KB_DT_BF16) KB_PRA(float, float, bf16);
    else return fail("proj_rope_append: dtype codes %d (input), %d (weights) -> %d are not handled", src_dt, w_dt, out_dt);
#undef KB_PRA
    return check_launch("proj_rope_append");
}

extern "C" int kb_pool_blocks(const void* k_table, const void* v_table, int dt, const int* block_table, int table_width, int n_pages,
                              const int* row_entry, const int* positions, const int* lines, const int* slots, float* pooled,
                              long long slot_stride, int n_slots, int max_blocks, int pool, int rows, int hkv, int d, int dv,
                              int page_size, void* stream) {
    KB_REQUIRE(rows >= 0 && hkv > 0 && d > 0 && dv > 0 && pool > 0 && max_blocks >= 0, "pool_blocks: rows %d, %d kv heads of %d / %d, blocks of %d", rows, hkv, d, dv, pool);
    KB_REQUIRE(table_width > 0 && n_pages > 0 && page_size > 0 && n_slots > 0, "pool_blocks: table width %d, pages %d of %d, slots %d", table_width, n_pages, page_size, n_slots);
    KB_REQUIRE(slot_stride >= (long long)max_blocks * hkv * (d + dv), "pool_blocks: a slot of %lld values for %d blocks", slot_stride, max_blocks);
    if (rows == 0 || max_blocks == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = hkv * (d + dv) >= 1024 ? 256 : 128;
    if (dt == KB_DT_F32)
        pool_blocks_kernel<float><<<rows, threads, 0, s>>>((const float*)k_table, (const float*)v_table, block_table, table_width, n_pages, row_entry,
                                                          positions, lines, slots, pooled, slot_stride, n_slots, max_blocks, pool, hkv, d, dv, page_size);
    else if (dt == KB_DT_BF16)
        pool_blocks_kernel<bf16><<<rows, threads, 0, s>>>((const bf16*)k_table, (const bf16*)v_table, block_table, table_width, n_pages, row_entry,
                                                         positions, lines, slots, pooled, slot_stride, n_slots, max_blocks, pool, hkv, d, dv, page_size);
    else return fail("pool_blocks: dtype code %d is not known", dt);
    return check_launch("pool_blocks");
}

// Scratch floats for `splits` slices of the keys (0 with one).
extern "C" long long kb_pooled_attention_scratch_floats(int rows, int hq, int dv, int splits, int split_keys) {
    return splits > 1 ? (long long)rows * splits * hq * (dv + 2 + split_keys) : 0;
}

extern "C" int kb_pooled_attention(void* out, const void* q, const void* k_table, const void* v_table, int dt, const float* pooled,
                                   long long slot_stride, int n_slots, int max_blocks, const int* block_table, const int* row_entry,
                                   const int* row_count, const int* slots, const float* talk, const float* temp, int rows, int hq,
                                   int hkv, int d, int dv, int page_size, int table_width, int n_pages, int window, int pool,
                                   float scale, int splits, int split_keys, float* scratch, void* stream) {
    KB_REQUIRE(rows >= 0 && hq > 0 && hkv > 0 && hq % hkv == 0 && d > 0 && dv > 0, "pooled_attention: rows %d, %d heads over %d, sizes %d / %d", rows, hq, hkv, d, dv);
    KB_REQUIRE(page_size > 0 && table_width > 0 && n_pages > 0, "pooled_attention: page_size %d, table width %d, pages %d", page_size, table_width, n_pages);
    KB_REQUIRE(window >= 0 && pool >= 0 && max_blocks >= 0, "pooled_attention: window %d, blocks of %d, %d blocks", window, pool, max_blocks);
    KB_REQUIRE(pool == 0 || (pooled != nullptr && n_slots > 0 && slot_stride >= (long long)max_blocks * hkv * (d + dv)),
               "pooled_attention: blocks of %d without a table that holds %d of them a slot", pool, max_blocks);
    KB_REQUIRE(splits >= 1 && splits <= 65535, "pooled_attention: %d slices", splits);
    KB_REQUIRE(splits == 1 || (scratch != nullptr && split_keys > 0 && split_keys % PA_CHUNK == 0), "pooled_attention: %d slices of %d keys", splits, split_keys);
    if (rows == 0) return 0;
    PooledParams p;
    p.q = q; p.k_table = k_table; p.v_table = v_table; p.pooled = pooled; p.block_table = block_table; p.row_entry = row_entry;
    p.row_count = row_count; p.slots = slots; p.talk = talk; p.temp = temp; p.out = out;
    p.stats = scratch; p.partial = scratch != nullptr ? scratch + (size_t)rows * splits * hq * 2 : nullptr;
    p.kept_scores = scratch != nullptr ? p.partial + (size_t)rows * splits * hq * dv : nullptr;
    p.slot_stride = slot_stride; p.rows = rows; p.hq = hq; p.hkv = hkv; p.d = d; p.dv = dv; p.page_size = page_size;
    p.table_width = table_width; p.n_pages = n_pages; p.n_slots = n_slots; p.max_blocks = max_blocks; p.window = window;
    p.pool = pool; p.splits = splits; p.split_keys = split_keys; p.mode = 0; p.scale = scale;
    cudaStream_t s = (cudaStream_t)stream;
    if (dt == KB_DT_F32) return run_pooled<float>(p, s);
    if (dt == KB_DT_BF16) return run_pooled<bf16>(p, s);
    return fail("pooled_attention: dtype code %d is not known", dt);
}
