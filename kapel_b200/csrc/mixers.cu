// What a mixer does around its products and its core, for mixers whose inputs come as one stacked
// product [rows, row_width] (a tensor or split-K partial sums) with each role at a column offset:
//
//  proj_norm_append  an RMS norm over the whole query projection and over the whole key projection
//                    (all heads' components of a row at once), the queries written out as
//                    [rows, hq, d], keys and values written to the paged cache at each row's line.
//                    The counterpart of rotate-and-append for a mixer without a rotation.
//  head_gate         y[r, h, :] (optionally divided by its root mean square over the head, times a
//                    weight over all heads) times sigmoid(gate[r, h, :]), the gate read from the
//                    stacked product; the output's rows may be wider than the heads (zeros behind them).
//  entry_ranges      first row and one past the last row of every request of a step, from the rows' entries.
//  head_norm_rope_append  an RMS norm over every head's query and key (a weight of the head's size,
//                    shared by the heads), then the rotation of the first `rotary` components, the
//                    queries written out, keys and values (of their own size) to the paged cache.
//  latent_append     for attention through latents: the query latent RMS-normed and written out; the
//                    key/value latent RMS-normed and, behind it, the one rotated key part of the row,
//                    written as the row's line of a cache with one kv head.
//  head_linear       y[r, h, :] = x[r, h, :] . M[h] for a matrix a head ([heads, n_in, n_out]); optionally
//                    a rotated copy of further components of x behind the product (the rotated part
//                    of a latent query), or sigmoid(gate) on the result. In 32-bit by FMA; with bfloat16
//                    matrices stored the other way round, on tensor cores (`head_linear_mma`).
//
// Sums, norms, rotations and the gates are 32-bit.
#include "common.cuh"

namespace kb {

typedef __nv_bfloat16 bf16;

template <typename TS, typename TW, typename TO>
__global__ void proj_norm_append_kernel(const Src<TS> src, int row_width, int q_off, int k_off, int v_off,
                                        const TW* __restrict__ wq, float eps_q, float off_q,
                                        const TW* __restrict__ wk, float eps_k, float off_k,
                                        const int* __restrict__ lines, TO* __restrict__ q_out, TO* __restrict__ k_table,
                                        TO* __restrict__ v_table, int hq, int hkv, int d, int dv, long long table_lines,
                                        int page_size) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const size_t base = (size_t)r * row_width;
    const int nq = hq * d, nk = hkv * d, nv = hkv * dv;
    float inv_q = 1.f, inv_k = 1.f;
    if (wq != nullptr) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < nq; i += blockDim.x) {
            const float v = src.at(base + q_off + i);
            ss += v * v;
        }
        ss = block_sum(ss, scratch);
        inv_q = 1.f / sqrtf(ss / (float)nq + eps_q);
    }
    if (wk != nullptr) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < nk; i += blockDim.x) {
            const float v = src.at(base + k_off + i);
            ss += v * v;
        }
        ss = block_sum(ss, scratch);
        inv_k = 1.f / sqrtf(ss / (float)nk + eps_k);
    }
    for (int i = threadIdx.x; i < nq; i += blockDim.x) {
        float v = src.at(base + q_off + i);
        if (wq != nullptr) v = v * inv_q * (off_q + Elem<TW>::load(wq + i));
        Elem<TO>::store(q_out + (size_t)r * nq + i, v);
    }
    if (k_table == nullptr) return;
    const long long line = lines[r];
    if (line < 0 || line >= table_lines) return;          // a row that writes nowhere (padding)
    for (int i = threadIdx.x; i < nk; i += blockDim.x) {
        float v = src.at(base + k_off + i);
        if (wk != nullptr) v = v * inv_k * (off_k + Elem<TW>::load(wk + i));
        const int h = i / d, c = i - h * d;
        Elem<TO>::store(k_table + kv_row(line, h, hkv, page_size) * d + c, v);
    }
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
        const int h = i / dv, c = i - h * dv;
        Elem<TO>::store(v_table + kv_row(line, h, hkv, page_size) * dv + c, src.at(base + v_off + i));
    }
}

// One warp a (row, head).
template <typename TY, typename TS, typename TW, typename TO>
__global__ void head_gate_kernel(TO* __restrict__ out, const TY* __restrict__ y, const Src<TS> gate, int row_width,
                                 int g_off, const TW* __restrict__ w, int unit, float eps, long long pairs, int heads, int e,
                                 int out_stride, int act) {
    const long long pair = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (pair >= pairs) return;
    const int lane = threadIdx.x & 31;
    const long long r = pair / heads;
    const int h = (int)(pair - r * heads);
    const TY* yp = y + (size_t)pair * e;
    float inv = 1.f;
    if (unit) {
        float ss = 0.f;
        for (int c = lane; c < e; c += 32) {
            const float v = Elem<TY>::load(yp + c);
            ss += v * v;
        }
        ss = warp_sum(ss);
        inv = 1.f / sqrtf(ss / (float)e + eps);
    }
    for (int c = lane; c < e; c += 32) {
        float v = Elem<TY>::load(yp + c) * inv;
        if (w != nullptr) v *= Elem<TW>::load(w + (size_t)h * e + c);
        if (act != 2) {                                                          // 2: no gate
            const float z = gate.at((size_t)r * row_width + g_off + (size_t)h * e + c);
            v *= act == 1 ? z / (1.f + expf(-z)) : 1.f / (1.f + expf(-z));       // silu(z) or sigmoid(z)
        }
        Elem<TO>::store(out + (size_t)r * out_stride + (size_t)h * e + c, v);
    }
    // a row wider than its heads (padding for the product that follows) ends in zeros
    if (h == heads - 1)
        for (int c = heads * e + lane; c < out_stride; c += 32) Elem<TO>::store(out + (size_t)r * out_stride + c, 0.f);
}

// One block a row; a warp takes head vectors in turn (queries, then keys, then values) through a
// piece of shared memory of its own.
template <typename TS, typename TW, typename TO>
__global__ void head_norm_rope_append_kernel(const Src<TS> src, int row_width, int q_off, int k_off, int v_off,
                                             const TW* __restrict__ wq, float eps_q, float off_q,
                                             const TW* __restrict__ wk, float eps_k, float off_k,
                                             const float2* __restrict__ cos_sin, int rotary,
                                             const int* __restrict__ lines, TO* __restrict__ q_out, TO* __restrict__ k_table,
                                             TO* __restrict__ v_table, int hq, int hkv, int d, int dv, long long table_lines,
                                             int page_size) {
    extern __shared__ float vecs[];                             // [warps][d]
    const int r = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    float* x = vecs + (size_t)warp * d;
    const size_t base = (size_t)r * row_width;
    const int half = rotary >> 1;
    long long line = -1;
    if (k_table != nullptr) {
        line = lines[r];
        if (line >= table_lines) line = -1;
    }
    for (int u = warp; u < hq + hkv; u += warps) {
        const bool is_q = u < hq;
        const int h = is_q ? u : u - hq;
        if (!is_q && line < 0) continue;                        // a row that writes nowhere
        const size_t at = base + (is_q ? q_off : k_off) + (size_t)h * d;
        const TW* w = is_q ? wq : wk;
        float ss = 0.f;
        for (int i = lane; i < d; i += 32) {
            const float v = src.at(at + i);
            x[i] = v;
            ss = fmaf(v, v, ss);
        }
        if (w != nullptr) {
            ss = warp_sum(ss);
            const float inv = 1.f / sqrtf(ss / (float)d + (is_q ? eps_q : eps_k));
            const float off = is_q ? off_q : off_k;
            for (int i = lane; i < d; i += 32) x[i] = x[i] * inv * (off + Elem<TW>::load(w + i));
        }
        __syncwarp();
        for (int i = lane; i < half; i += 32) {
            float a = x[i], b = x[i + half];
            rope_rotate(a, b, cos_sin[(size_t)r * half + i]);
            x[i] = a;
            x[i + half] = b;
        }
        __syncwarp();
        TO* dst = is_q ? q_out + ((size_t)r * hq + h) * d : k_table + kv_row(line, h, hkv, page_size) * d;
        for (int i = lane; i < d; i += 32) Elem<TO>::store(dst + i, x[i]);
        __syncwarp();
    }
    if (line < 0) return;
    for (int i = threadIdx.x; i < hkv * dv; i += blockDim.x) {
        const int h = i / dv, c = i - h * dv;
        Elem<TO>::store(v_table + kv_row(line, h, hkv, page_size) * dv + c, src.at(base + v_off + i));
    }
}

// One block a row. The cache has one kv head whose line is [latent (kv_rank) | rotated part (rot)].
template <typename TS, typename TW, typename TO>
__global__ void latent_append_kernel(const Src<TS> src, int row_width, int q_off, int kv_off, int q_rank, int kv_rank, int rot,
                                     const TW* __restrict__ wq, const TW* __restrict__ wkv, float eps,
                                     const float2* __restrict__ cos_sin, const int* __restrict__ lines,
                                     TO* __restrict__ cq_out, int cq_stride, TO* __restrict__ k_table, long long table_lines,
                                     int page_size) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const size_t base = (size_t)r * row_width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
        const float v = src.at(base + q_off + i);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv_q = 1.f / sqrtf(ss / (float)q_rank + eps);
    for (int i = threadIdx.x; i < cq_stride; i += blockDim.x) {
        const float v = i < q_rank ? src.at(base + q_off + i) * inv_q * Elem<TW>::load(wq + i) : 0.f;
        Elem<TO>::store(cq_out + (size_t)r * cq_stride + i, v);
    }
    if (k_table == nullptr) return;
    const long long line = lines[r];
    if (line < 0 || line >= table_lines) return;                // a row that writes nowhere (padding)
    float sk = 0.f;
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) {
        const float v = src.at(base + kv_off + i);
        sk = fmaf(v, v, sk);
    }
    sk = block_sum(sk, scratch);
    const float inv_k = 1.f / sqrtf(sk / (float)kv_rank + eps);
    TO* dst = k_table + kv_row(line, 0, 1, page_size) * (kv_rank + rot);
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x)
        Elem<TO>::store(dst + i, src.at(base + kv_off + i) * inv_k * Elem<TW>::load(wkv + i));
    const int half = rot >> 1;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float a = src.at(base + kv_off + kv_rank + i), b = src.at(base + kv_off + kv_rank + i + half);
        rope_rotate(a, b, cos_sin[(size_t)r * half + i]);
        Elem<TO>::store(dst + kv_rank + i, a);
        Elem<TO>::store(dst + kv_rank + i + half, b);
    }
}

// y[r, h, c] = sum_i x[r, h, i] M[h, i, c]. One block = HL_ROWS rows x one head x HL_COLS columns; the rows'
// inputs lie in shared memory, a thread owns a column and walks M[h, :, c] (neighbours read neighbours).
constexpr int HL_ROWS = 8;
constexpr int HL_COLS = 128;
template <typename TX, typename T>
__global__ void __launch_bounds__(HL_COLS)
head_linear_kernel(T* __restrict__ y, int y_row, int y_head, const Src<TX> x, int x_row, int x_head, int x_off,
                   const T* __restrict__ m, int n_in, int n_out, int rows, int heads,
                   int tail_off, int tail, const float2* __restrict__ cos_sin,
                   const Src<float> gate, int g_row, int g_off) {
    extern __shared__ float xs[];                               // [HL_ROWS][n_in]
    const int rbase = blockIdx.x * HL_ROWS, h = blockIdx.y;
    const int nr = min(HL_ROWS, rows - rbase);
    for (int idx = threadIdx.x; idx < HL_ROWS * n_in; idx += HL_COLS) {
        const int t = idx / n_in, i = idx - t * n_in;
        xs[idx] = t < nr ? x.at((size_t)(rbase + t) * x_row + (size_t)h * x_head + x_off + i) : 0.f;
    }
    __syncthreads();
    const int c = blockIdx.z * HL_COLS + threadIdx.x;
    if (c < n_out) {
        float acc[HL_ROWS];
#pragma unroll
        for (int t = 0; t < HL_ROWS; ++t) acc[t] = 0.f;
        const T* col = m + (size_t)h * n_in * n_out + c;
        int i = 0;
        for (; i + 4 <= n_in; i += 4) {                         // four loads in flight
            float w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Elem<T>::load(col + (size_t)(i + j) * n_out);
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int t = 0; t < HL_ROWS; ++t) acc[t] = fmaf(xs[t * n_in + i + j], w[j], acc[t]);
        }
        for (; i < n_in; ++i) {
            const float w = Elem<T>::load(col + (size_t)i * n_out);
#pragma unroll
            for (int t = 0; t < HL_ROWS; ++t) acc[t] = fmaf(xs[t * n_in + i], w, acc[t]);
        }
#pragma unroll
        for (int t = 0; t < HL_ROWS; ++t) {
            if (t >= nr) continue;
            float v = acc[t];
            if (gate.p != nullptr) {
                const float z = gate.at((size_t)(rbase + t) * g_row + g_off + (size_t)h * n_out + c);
                v *= 1.f / (1.f + expf(-z));
            }
            Elem<T>::store(y + (size_t)(rbase + t) * y_row + (size_t)h * y_head + c, v);
        }
    }
    if (blockIdx.z != 0) return;
    // behind the product: `tail` further components of x, rotated
    const int half = tail >> 1;
    for (int idx = threadIdx.x; idx < nr * half; idx += HL_COLS) {
        const int t = idx / half, i = idx - t * half;
        const size_t at = (size_t)(rbase + t) * x_row + (size_t)h * x_head + tail_off;
        float a = x.at(at + i), b = x.at(at + i + half);
        rope_rotate(a, b, cos_sin[(size_t)(rbase + t) * half + i]);
        T* dst = y + (size_t)(rbase + t) * y_row + (size_t)h * y_head + n_out;
        Elem<T>::store(dst + i, a);
        Elem<T>::store(dst + i + half, b);
    }
    // a row wider than its heads (padding for the product that follows) ends in zeros
    if (h == heads - 1)
        for (int idx = threadIdx.x; idx < nr * (y_row - heads * y_head); idx += HL_COLS) {
            const int pad = y_row - heads * y_head;
            const int t = idx / pad, i = idx - t * pad;
            Elem<T>::store(y + (size_t)(rbase + t) * y_row + heads * y_head + i, 0.f);
        }
}

// The same product on tensor cores (mma.sync m16n8k16, bfloat16 in, 32-bit sums) with the matrices stored
// the other way round, mt [heads, n_out, n_in] (a column of M[h] lies together, as the B operand wants it).
// One block = 64 rows x one head x 64 columns, four warps of 16 rows; the inner dimension 32 at a time through
// shared memory (the inputs rounded to bfloat16 there). Any sizes: what lies beyond an edge is zero.
constexpr int HM_ROWS = 64;
constexpr int HM_COLS = 64;
constexpr int HM_K = 32;
constexpr int HM_LD = HM_K + 8;
template <typename TX>
__global__ void __launch_bounds__(128)
head_linear_mma_kernel(bf16* __restrict__ y, int y_row, int y_head, const Src<TX> x, int x_row, int x_head, int x_off,
                       const bf16* __restrict__ mt, int n_in, int n_out, int rows, int heads,
                       int tail_off, int tail, const float2* __restrict__ cos_sin,
                       const Src<float> gate, int g_row, int g_off) {
    __shared__ __align__(16) bf16 sa[HM_ROWS * HM_LD];
    __shared__ __align__(16) bf16 sb[HM_COLS * HM_LD];
    const int rbase = blockIdx.x * HM_ROWS, h = blockIdx.y, cbase = blockIdx.z * HM_COLS;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, t4 = lane & 3;
    float acc[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
    const bool wide = n_in % 8 == 0 && ((uintptr_t)mt & 15) == 0;
    for (int k0 = 0; k0 < n_in; k0 += HM_K) {
        for (int idx = tid; idx < HM_ROWS * HM_K; idx += 128) {
            const int r = idx / HM_K, k = idx - r * HM_K;
            float v = 0.f;
            if (rbase + r < rows && k0 + k < n_in) v = x.at((size_t)(rbase + r) * x_row + (size_t)h * x_head + x_off + k0 + k);
            sa[r * HM_LD + k] = __float2bfloat16_rn(v);
        }
        if (wide) {
            for (int idx = tid; idx < HM_COLS * (HM_K / 8); idx += 128) {
                const int n = idx / (HM_K / 8), v = idx - n * (HM_K / 8);
                uint4 val = make_uint4(0u, 0u, 0u, 0u);
                if (cbase + n < n_out && k0 + v * 8 < n_in)
                    val = *reinterpret_cast<const uint4*>(mt + ((size_t)h * n_out + cbase + n) * n_in + k0 + v * 8);
                *reinterpret_cast<uint4*>(sb + n * HM_LD + v * 8) = val;
            }
        } else {
            for (int idx = tid; idx < HM_COLS * HM_K; idx += 128) {
                const int n = idx / HM_K, k = idx - n * HM_K;
                sb[n * HM_LD + k] = (cbase + n < n_out && k0 + k < n_in) ? mt[((size_t)h * n_out + cbase + n) * n_in + k0 + k] : __float2bfloat16_rn(0.f);
            }
        }
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < HM_K; ks += 16) {
            const bf16* pa = sa + (warp * 16 + gid) * HM_LD + ks + 2 * t4;
            const uint32_t a0 = *reinterpret_cast<const uint32_t*>(pa), a1 = *reinterpret_cast<const uint32_t*>(pa + 8 * HM_LD);
            const uint32_t a2 = *reinterpret_cast<const uint32_t*>(pa + 8), a3 = *reinterpret_cast<const uint32_t*>(pa + 8 * HM_LD + 8);
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                const bf16* pb = sb + (nt * 8 + gid) * HM_LD + ks + 2 * t4;
                const uint32_t b0 = *reinterpret_cast<const uint32_t*>(pb), b1 = *reinterpret_cast<const uint32_t*>(pb + 8);
                asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                             : "+f"(acc[nt][0]), "+f"(acc[nt][1]), "+f"(acc[nt][2]), "+f"(acc[nt][3])
                             : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = rbase + warp * 16 + gid + 8 * (i >> 1), c = cbase + nt * 8 + 2 * t4 + (i & 1);
            if (r >= rows || c >= n_out) continue;
            float v = acc[nt][i];
            if (gate.p != nullptr) {
                const float z = gate.at((size_t)r * g_row + g_off + (size_t)h * n_out + c);
                v *= 1.f / (1.f + expf(-z));
            }
            y[(size_t)r * y_row + (size_t)h * y_head + c] = __float2bfloat16_rn(v);
        }
    }
    if (blockIdx.z != 0) return;
    const int nr = min(HM_ROWS, rows - rbase);
    const int half = tail >> 1;
    for (int idx = tid; idx < nr * half; idx += 128) {          // behind the product: `tail` further components of x, rotated
        const int t = idx / half, i = idx - t * half;
        const size_t at = (size_t)(rbase + t) * x_row + (size_t)h * x_head + tail_off;
        float a = x.at(at + i), b = x.at(at + i + half);
        rope_rotate(a, b, cos_sin[(size_t)(rbase + t) * half + i]);
        bf16* dst = y + (size_t)(rbase + t) * y_row + (size_t)h * y_head + n_out;
        dst[i] = __float2bfloat16_rn(a);
        dst[i + half] = __float2bfloat16_rn(b);
    }
    if (h == heads - 1) {                                       // a row wider than its heads ends in zeros
        const int pad = y_row - heads * y_head;
        for (int idx = tid; idx < nr * pad; idx += 128) {
            const int t = idx / pad, i = idx - t * pad;
            y[(size_t)(rbase + t) * y_row + heads * y_head + i] = __float2bfloat16_rn(0.f);
        }
    }
}

// The same product for a few rows (a decode step): one warp a column of M[h] for all rows. The lanes walk the
// column's n_in values (they lie together in mt [heads, n_out, n_in]), every row's inputs lie in shared memory;
// a warp sum a row. 32-bit sums; inputs and matrices as they come (no rounding of the inputs).
constexpr int HF_ROWS = 16;
constexpr int HF_WARPS = 8;
template <typename TX>
__global__ void __launch_bounds__(HF_WARPS * 32)
head_linear_few_kernel(bf16* __restrict__ y, int y_row, int y_head, const Src<TX> x, int x_row, int x_head, int x_off,
                       const bf16* __restrict__ mt, int n_in, int n_out, int rows, int heads,
                       int tail_off, int tail, const float2* __restrict__ cos_sin,
                       const Src<float> gate, int g_row, int g_off) {
    extern __shared__ float xf[];                               // [rows][n_in]
    const int h = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int idx = tid; idx < rows * n_in; idx += HF_WARPS * 32) {
        const int t = idx / n_in, i = idx - t * n_in;
        xf[idx] = x.at((size_t)t * x_row + (size_t)h * x_head + x_off + i);
    }
    __syncthreads();
    const int c = blockIdx.y * HF_WARPS + warp;
    if (c < n_out) {
        float acc[HF_ROWS];
#pragma unroll
        for (int t = 0; t < HF_ROWS; ++t) acc[t] = 0.f;
        const bf16* col = mt + ((size_t)h * n_out + c) * n_in;
        for (int i = lane; i < n_in; i += 32) {
            const float w = __bfloat162float(col[i]);
#pragma unroll
            for (int t = 0; t < HF_ROWS; ++t)
                if (t < rows) acc[t] = fmaf(xf[t * n_in + i], w, acc[t]);
        }
#pragma unroll
        for (int t = 0; t < HF_ROWS; ++t) {
            if (t >= rows) continue;
            float v = warp_sum(acc[t]);
            if (lane == 0) {
                if (gate.p != nullptr) {
                    const float z = gate.at((size_t)t * g_row + g_off + (size_t)h * n_out + c);
                    v *= 1.f / (1.f + expf(-z));
                }
                y[(size_t)t * y_row + (size_t)h * y_head + c] = __float2bfloat16_rn(v);
            }
        }
    }
    if (blockIdx.y != 0) return;
    const int half = tail >> 1;
    for (int idx = tid; idx < rows * half; idx += HF_WARPS * 32) {
        const int t = idx / half, i = idx - t * half;
        const size_t at = (size_t)t * x_row + (size_t)h * x_head + tail_off;
        float a = x.at(at + i), b = x.at(at + i + half);
        rope_rotate(a, b, cos_sin[(size_t)t * half + i]);
        bf16* dst = y + (size_t)t * y_row + (size_t)h * y_head + n_out;
        dst[i] = __float2bfloat16_rn(a);
        dst[i + half] = __float2bfloat16_rn(b);
    }
    if (h == heads - 1) {
        const int pad = y_row - heads * y_head;
        for (int idx = tid; idx < rows * pad; idx += HF_WARPS * 32) {
            const int t = idx / pad, i = idx - t * pad;
            y[(size_t)t * y_row + heads * y_head + i] = __float2bfloat16_rn(0.f);
        }
    }
}

__global__ void entry_ranges_clear_kernel(int entries, int* __restrict__ start, int* __restrict__ end) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < entries) {                                      // an entry without rows keeps the empty range
        start[i] = 0;
        end[i] = 0;
    }
}
__global__ void entry_ranges_fill_kernel(const int* __restrict__ row_entry, int rows, int entries, int* __restrict__ start,
                                         int* __restrict__ end) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    const int e = row_entry[r];
    if (e < 0 || e >= entries) return;
    if (r == 0 || row_entry[r - 1] != e) start[e] = r;
    if (r == rows - 1 || row_entry[r + 1] != e) end[e] = r + 1;
}

}  // namespace kb

using namespace kb;

// Rows [start[e], end[e]) are entry e's (the rows of one entry lie together). Two launches.
extern "C" int kb_entry_ranges(int* start, int* end, const int* row_entry, int rows, int entries, void* stream) {
    KB_REQUIRE(rows >= 0 && entries >= 0, "entry_ranges: rows %d, entries %d", rows, entries);
    if (entries == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    entry_ranges_clear_kernel<<<(entries + 255) / 256, 256, 0, s>>>(entries, start, end);
    if (int e = check_launch("entry_ranges")) return e;
    if (rows == 0) return 0;
    entry_ranges_fill_kernel<<<(rows + 255) / 256, 256, 0, s>>>(row_entry, rows, entries, start, end);
    return check_launch("entry_ranges");
}

extern "C" int kb_proj_norm_append(const void* src, int in_dt, int splits, long long split_stride, int row_width, int q_off,
                                   int k_off, int v_off, const void* wq, float eps_q, float off_q, const void* wk,
                                   float eps_k, float off_k, int w_dt, const int* lines, void* q_out, void* k_table,
                                   void* v_table, int out_dt, int rows, int hq, int hkv, int d, int dv, int write_kv,
                                   long long table_lines, int page_size, void* stream) {
    KB_REQUIRE(rows >= 0 && hq > 0 && hkv > 0 && d > 0 && dv > 0, "proj_norm_append: rows %d, heads %d / %d, sizes %d / %d", rows, hq, hkv, d, dv);
    KB_REQUIRE(row_width > 0 && q_off >= 0 && q_off + hq * d <= row_width && k_off >= 0 && k_off + hkv * d <= row_width &&
                   v_off >= 0 && v_off + hkv * dv <= row_width,
               "proj_norm_append: columns q %d, k %d, v %d do not fit a row of %d", q_off, k_off, v_off, row_width);
    KB_REQUIRE(splits >= 1 && (splits == 1 || split_stride >= (long long)rows * row_width), "proj_norm_append: %d slices %lld apart", splits, split_stride);
    KB_REQUIRE(!write_kv || (lines && k_table && v_table && table_lines > 0 && page_size > 0), "proj_norm_append: no cache to write");
    if (rows == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    void* kt = write_kv ? k_table : nullptr;
    const int threads = 256;
#define KB_PNA(TS, TW, TO)                                                                                              \
    proj_norm_append_kernel<TS, TW, TO><<<rows, threads, 0, s>>>(Src<TS>{(const TS*)src, splits, (size_t)split_stride}, row_width, q_off, \
                                                                 k_off, v_off, (const TW*)wq, eps_q, off_q, (const TW*)wk, eps_k, off_k, \
                                                                 lines, (TO*)q_out, (TO*)kt, (TO*)v_table, hq, hkv, d, dv, table_lines, page_size)
    const int code = in_dt * 4 + w_dt * 2 + out_dt;
    switch (code) {
        case 0: KB_PNA(float, float, float); break;
        case 1: KB_PNA(float, float, bf16); break;
        case 2: KB_PNA(float, bf16, float); break;
        case 3: KB_PNA(float, bf16, bf16); break;
        case 4: KB_PNA(bf16, float, float); break;
        case 5: KB_PNA(bf16, float, bf16); break;
        case 6: KB_PNA(bf16, bf16, float); break;
        case 7: KB_PNA(bf16, bf16, bf16); break;
        default: return fail("proj_norm_append: dtype codes in %d, w %d, out %d are not known", in_dt, w_dt, out_dt);
    }
#undef KB_PNA
    return check_launch("proj_norm_append");
}

extern "C" int kb_head_gate(void* out, int out_dt, const void* y, int y_dt, const void* gate, int g_dt, int splits,
                            long long split_stride, int row_width, int g_off, const void* w, int w_dt, int unit, float eps,
                            long long rows, int heads, int e, int out_stride, int act, void* stream) {
    KB_REQUIRE(rows >= 0 && heads > 0 && e > 0, "head_gate: rows %lld, heads %d of %d", rows, heads, e);
    KB_REQUIRE(act >= 0 && act <= 2, "head_gate: gate activation code %d is not known (0 sigmoid, 1 silu, 2 none)", act);
    KB_REQUIRE(out_stride >= heads * e, "head_gate: output rows of %d values for %d heads of %d", out_stride, heads, e);
    KB_REQUIRE(row_width > 0 && g_off >= 0 && g_off + heads * e <= row_width, "head_gate: gate columns %d.. do not fit a row of %d", g_off, row_width);
    KB_REQUIRE(splits >= 1 && (splits == 1 || split_stride >= rows * row_width), "head_gate: %d slices %lld apart", splits, split_stride);
    if (rows == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const long long pairs = rows * heads;
    const int warps = 4;
    const long long blocks = (pairs + warps - 1) / warps;
    KB_REQUIRE(blocks <= 0x7fffffffll, "head_gate: too many rows for one launch");
#define KB_HG(TY, TS, TW, TO)                                                                                       \
    head_gate_kernel<TY, TS, TW, TO><<<(unsigned)blocks, warps * 32, 0, s>>>((TO*)out, (const TY*)y,                    \
                                                                             Src<TS>{(const TS*)gate, splits, (size_t)split_stride}, \
                                                                             row_width, g_off, (const TW*)w, unit, eps, pairs, heads, e, out_stride, act)
    const int code = y_dt * 8 + g_dt * 4 + w_dt * 2 + out_dt;
    switch (code) {
        case 0: KB_HG(float, float, float, float); break;
        case 1: KB_HG(float, float, float, bf16); break;
        case 2: KB_HG(float, float, bf16, float); break;
        case 3: KB_HG(float, float, bf16, bf16); break;
        case 4: KB_HG(float, bf16, float, float); break;
        case 5: KB_HG(float, bf16, float, bf16); break;
        case 6: KB_HG(float, bf16, bf16, float); break;
        case 7: KB_HG(float, bf16, bf16, bf16); break;
        case 8: KB_HG(bf16, float, float, float); break;
        case 9: KB_HG(bf16, float, float, bf16); break;
        case 10: KB_HG(bf16, float, bf16, float); break;
        case 11: KB_HG(bf16, float, bf16, bf16); break;
        case 12: KB_HG(bf16, bf16, float, float); break;
        case 13: KB_HG(bf16, bf16, float, bf16); break;
        case 14: KB_HG(bf16, bf16, bf16, float); break;
        case 15: KB_HG(bf16, bf16, bf16, bf16); break;
        default: return fail("head_gate: dtype codes y %d, gate %d, w %d, out %d are not known", y_dt, g_dt, w_dt, out_dt);
    }
#undef KB_HG
    return check_launch("head_gate");
}

extern "C" int kb_head_norm_rope_append(const void* src, int in_dt, int splits, long long split_stride, int row_width, int q_off,
                                        int k_off, int v_off, const void* wq, float eps_q, float off_q, const void* wk,
                                        float eps_k, float off_k, int w_dt, const float* cos_sin, int rotary, const int* lines,
                                        void* q_out, void* k_table, void* v_table, int out_dt, int rows, int hq, int hkv, int d,
                                        int dv, int write_kv, long long table_lines, int page_size, void* stream) {
    KB_REQUIRE(rows >= 0 && hq > 0 && hkv > 0 && d > 0 && dv > 0, "head_norm_rope_append: rows %d, heads %d / %d, sizes %d / %d", rows, hq, hkv, d, dv);
    KB_REQUIRE(rotary >= 0 && rotary <= d && rotary % 2 == 0, "head_norm_rope_append: rotary %d must be even and at most the head's %d", rotary, d);
    KB_REQUIRE(rotary == 0 || cos_sin != nullptr, "head_norm_rope_append: a rotation without its table");
    KB_REQUIRE(row_width > 0 && q_off >= 0 && q_off + hq * d <= row_width && k_off >= 0 && k_off + hkv * d <= row_width &&
                   v_off >= 0 && v_off + hkv * dv <= row_width,
               "head_norm_rope_append: columns q %d, k %d, v %d do not fit a row of %d", q_off, k_off, v_off, row_width);
    KB_REQUIRE(splits >= 1 && (splits == 1 || split_stride >= (long long)rows * row_width), "head_norm_rope_append: %d slices %lld apart", splits, split_stride);
    KB_REQUIRE(!write_kv || (lines && k_table && v_table && table_lines > 0 && page_size > 0), "head_norm_rope_append: no cache to write");
    KB_REQUIRE(d <= 4096, "head_norm_rope_append: a head of %d components", d);
    if (rows == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    void* kt = write_kv ? k_table : nullptr;
    const int warps = rows <= DEPENDENT_ROWS ? 16 : 4;          // few rows: a head vector a warp side by side
    const size_t smem = (size_t)warps * d * sizeof(float);
#define KB_HNRA(TS, TW, TO)                                                                                              \
    head_norm_rope_append_kernel<TS, TW, TO><<<rows, warps * 32, smem, s>>>(                                                 \
        Src<TS>{(const TS*)src, splits, (size_t)split_stride}, row_width, q_off, k_off, v_off, (const TW*)wq, eps_q, off_q,  \
        (const TW*)wk, eps_k, off_k, (const float2*)cos_sin, rotary, lines, (TO*)q_out, (TO*)kt, (TO*)v_table, hq, hkv, d, dv, \
        table_lines, page_size)
    const int code = in_dt * 4 + w_dt * 2 + out_dt;
    switch (code) {
        case 0: KB_HNRA(float, float, float); break;
        case 1: KB_HNRA(float, float, bf16); break;
        case 2: KB_HNRA(float, bf16, float); break;
        case 3: KB_HNRA(float, bf16, bf16); break;
        case 4: KB_HNRA(bf16, float, float); break;
        case 5: KB_HNRA(bf16, float, bf16); break;
        case 6: KB_HNRA(bf16, bf16, float); break;
        case 7: KB_HNRA(bf16, bf16, bf16); break;
        default: return fail("head_norm_rope_append: dtype codes in %d, w %d, out %d are not known", in_dt, w_dt, out_dt);
    }
#undef KB_HNRA
    return check_launch("head_norm_rope_append");
}

extern "C" int kb_latent_append(const void* src, int in_dt, int splits, long long split_stride, int row_width, int q_off, int kv_off,
                                int q_rank, int kv_rank, int rot, const void* wq, const void* wkv, int w_dt, float eps,
                                const float* cos_sin, const int* lines, void* cq_out, int cq_stride, void* k_table, int out_dt,
                                int rows, int write_kv, long long table_lines, int page_size, void* stream) {
    KB_REQUIRE(rows >= 0 && q_rank > 0 && kv_rank > 0 && rot >= 0 && rot % 2 == 0, "latent_append: rows %d, ranks %d / %d, rotated %d", rows, q_rank, kv_rank, rot);
    KB_REQUIRE(row_width > 0 && q_off >= 0 && q_off + q_rank <= row_width && kv_off >= 0 && kv_off + kv_rank + rot <= row_width,
               "latent_append: columns q %d, kv %d do not fit a row of %d", q_off, kv_off, row_width);
    KB_REQUIRE(splits >= 1 && (splits == 1 || split_stride >= (long long)rows * row_width), "latent_append: %d slices %lld apart", splits, split_stride);
    KB_REQUIRE(cq_stride >= q_rank && wq && wkv && cq_out, "latent_append: output rows of %d for a latent of %d, or a weight is missing", cq_stride, q_rank);
    KB_REQUIRE(rot == 0 || cos_sin != nullptr, "latent_append: a rotation without its table");
    KB_REQUIRE(!write_kv || (lines && k_table && table_lines > 0 && page_size > 0), "latent_append: no cache to write");
    if (rows == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    void* kt = write_kv ? k_table : nullptr;
#define KB_LA(TS, TW, TO)                                                                                                  \
    latent_append_kernel<TS, TW, TO><<<rows, rows <= DEPENDENT_ROWS ? 1024 : 128, 0, s>>>(Src<TS>{(const TS*)src, splits, (size_t)split_stride}, row_width, q_off, \
                                                          kv_off, q_rank, kv_rank, rot, (const TW*)wq, (const TW*)wkv, eps,     \
                                                          (const float2*)cos_sin, lines, (TO*)cq_out, cq_stride, (TO*)kt,       \
                                                          table_lines, page_size)
    const int code = in_dt * 4 + w_dt * 2 + out_dt;
    switch (code) {
        case 0: KB_LA(float, float, float); break;
        case 1: KB_LA(float, float, bf16); break;
        case 2: KB_LA(float, bf16, float); break;
        case 3: KB_LA(float, bf16, bf16); break;
        case 4: KB_LA(bf16, float, float); break;
        case 5: KB_LA(bf16, float, bf16); break;
        case 6: KB_LA(bf16, bf16, float); break;
        case 7: KB_LA(bf16, bf16, bf16); break;
        default: return fail("latent_append: dtype codes in %d, w %d, out %d are not known", in_dt, w_dt, out_dt);
    }
#undef KB_LA
    return check_launch("latent_append");
}

// x: `x_dt`, maybe split-K partial sums; m and y: `dt`; gate: float32 (maybe partial sums) or null.
extern "C" int kb_head_linear(void* y, int dt, int y_row, int y_head, const void* x, int x_dt, int x_splits, long long x_split_stride,
                              int x_row, int x_head, int x_off, const void* m, int n_in, int n_out, int rows, int heads,
                              int tail_off, int tail, const float* cos_sin, const float* gate, int g_splits,
                              long long g_split_stride, int g_row, int g_off, void* stream) {
    KB_REQUIRE(rows >= 0 && heads > 0 && n_in > 0 && n_out > 0, "head_linear: rows %d, heads %d, sizes %d -> %d", rows, heads, n_in, n_out);
    KB_REQUIRE(tail >= 0 && tail % 2 == 0 && (tail == 0 || cos_sin != nullptr), "head_linear: %d rotated components (even, with a table)", tail);
    KB_REQUIRE(y_head >= n_out + tail && y_row >= heads * y_head, "head_linear: output rows of %d, heads of %d for %d + %d values", y_row, y_head, n_out, tail);
    KB_REQUIRE(x_off >= 0 && x_off + n_in <= x_head && (tail == 0 || (tail_off >= 0 && tail_off + tail <= x_head)) && x_row >= heads * x_head,
               "head_linear: input rows of %d, heads of %d, columns %d.. and %d..", x_row, x_head, x_off, tail_off);
    KB_REQUIRE(x_splits >= 1 && (x_splits == 1 || x_split_stride >= (long long)rows * x_row), "head_linear: %d slices %lld apart", x_splits, x_split_stride);
    KB_REQUIRE(gate == nullptr || (g_splits >= 1 && g_off >= 0 && g_off + heads * n_out <= g_row), "head_linear: gate columns %d.. of a row of %d", g_off, g_row);
    const size_t smem = (size_t)HL_ROWS * n_in * sizeof(float);
    KB_REQUIRE(smem <= 200 * 1024, "head_linear: %d inputs a head do not fit the shared memory of a block", n_in);
    KB_REQUIRE(heads <= 65535 && (n_out + HL_COLS - 1) / HL_COLS <= 65535, "head_linear: too many heads or columns for one launch");
    if (rows == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid((rows + HL_ROWS - 1) / HL_ROWS, heads, (n_out + HL_COLS - 1) / HL_COLS);
    const Src<float> g{gate, gate ? g_splits : 1, (size_t)g_split_stride};
#define KB_HL(TX, T)                                                                                                       \
    do {                                                                                                                   \
        if (smem > 48 * 1024) cudaFuncSetAttribute(head_linear_kernel<TX, T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        head_linear_kernel<TX, T><<<grid, HL_COLS, smem, s>>>((T*)y, y_row, y_head, Src<TX>{(const TX*)x, x_splits, (size_t)x_split_stride}, \
                                                            x_row, x_head, x_off, (const T*)m, n_in, n_out, rows, heads, tail_off, \
                                                            tail, (const float2*)cos_sin, g, g_row, g_off);                 \
    } while (0)
    const int code = x_dt * 2 + dt;
    switch (code) {
        case 0: KB_HL(float, float); break;
        case 1: KB_HL(float, bf16); break;
        case 2: KB_HL(bf16, float); break;
        case 3: KB_HL(bf16, bf16); break;
        default: return fail("head_linear: dtype codes x %d, weights %d are not known", x_dt, dt);
    }
#undef KB_HL
    return check_launch("head_linear");
}

// As kb_head_linear with bfloat16 matrices stored [heads, n_out, n_in], on tensor cores; y is bfloat16.
extern "C" int kb_head_linear_mma(void* y, int y_row, int y_head, const void* x, int x_dt, int x_splits, long long x_split_stride,
                                  int x_row, int x_head, int x_off, const void* mt, int n_in, int n_out, int rows, int heads,
                                  int tail_off, int tail, const float* cos_sin, const float* gate, int g_splits,
                                  long long g_split_stride, int g_row, int g_off, void* stream) {
    KB_REQUIRE(rows >= 0 && heads > 0 && n_in > 0 && n_out > 0, "head_linear_mma: rows %d, heads %d, sizes %d -> %d", rows, heads, n_in, n_out);
    KB_REQUIRE(tail >= 0 && tail % 2 == 0 && (tail == 0 || cos_sin != nullptr), "head_linear_mma: %d rotated components (even, with a table)", tail);
    KB_REQUIRE(y_head >= n_out + tail && y_row >= heads * y_head, "head_linear_mma: output rows of %d, heads of %d for %d + %d values", y_row, y_head, n_out, tail);
    KB_REQUIRE(x_off >= 0 && x_off + n_in <= x_head && (tail == 0 || (tail_off >= 0 && tail_off + tail <= x_head)) && x_row >= heads * x_head,
               "head_linear_mma: input rows of %d, heads of %d, columns %d.. and %d..", x_row, x_head, x_off, tail_off);
    KB_REQUIRE(x_splits >= 1 && (x_splits == 1 || x_split_stride >= (long long)rows * x_row), "head_linear_mma: %d slices %lld apart", x_splits, x_split_stride);
    KB_REQUIRE(gate == nullptr || (g_splits >= 1 && g_off >= 0 && g_off + heads * n_out <= g_row), "head_linear_mma: gate columns %d.. of a row of %d", g_off, g_row);
    KB_REQUIRE(heads <= 65535 && (n_out + HM_COLS - 1) / HM_COLS <= 65535, "head_linear_mma: too many heads or columns for one launch");
    if (rows == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const Src<float> g{gate, gate ? g_splits : 1, (size_t)g_split_stride};
    const size_t few_smem = (size_t)rows * n_in * sizeof(float);
    if (rows <= HF_ROWS && few_smem <= 48 * 1024 && (n_out + HF_WARPS - 1) / HF_WARPS <= 65535) {     // a decode step: a warp a column
        dim3 few(heads, (n_out + HF_WARPS - 1) / HF_WARPS);
        if (x_dt == KB_DT_F32)
            head_linear_few_kernel<float><<<few, HF_WARPS * 32, few_smem, s>>>((bf16*)y, y_row, y_head, Src<float>{(const float*)x, x_splits, (size_t)x_split_stride}, x_row,
                                                                             x_head, x_off, (const bf16*)mt, n_in, n_out, rows, heads, tail_off, tail, (const float2*)cos_sin, g, g_row, g_off);
        else if (x_dt == KB_DT_BF16)
            head_linear_few_kernel<bf16><<<few, HF_WARPS * 32, few_smem, s>>>((bf16*)y, y_row, y_head, Src<bf16>{(const bf16*)x, x_splits, (size_t)x_split_stride}, x_row,
                                                                            x_head, x_off, (const bf16*)mt, n_in, n_out, rows, heads, tail_off, tail, (const float2*)cos_sin, g, g_row, g_off);
        else return fail("head_linear_mma: dtype code %d is not known", x_dt);
        return check_launch("head_linear_few");
    }
    dim3 grid((rows + HM_ROWS - 1) / HM_ROWS, heads, (n_out + HM_COLS - 1) / HM_COLS);
    if (x_dt == KB_DT_F32)
        head_linear_mma_kernel<float><<<grid, 128, 0, s>>>((bf16*)y, y_row, y_head, Src<float>{(const float*)x, x_splits, (size_t)x_split_stride}, x_row, x_head,
                                                          x_off, (const bf16*)mt, n_in, n_out, rows, heads, tail_off, tail, (const float2*)cos_sin, g, g_row, g_off);
    else if (x_dt == KB_DT_BF16)
        head_linear_mma_kernel<bf16><<<grid, 128, 0, s>>>((bf16*)y, y_row, y_head, Src<bf16>{(const bf16*)x, x_splits, (size_t)x_split_stride}, x_row, x_head,
                                                         x_off, (const bf16*)mt, n_in, n_out, rows, heads, tail_off, tail, (const float2*)cos_sin, g, g_row, g_off);
    else return fail("head_linear_mma: dtype code %d is not known", x_dt);
    return check_launch("head_linear_mma");
}
