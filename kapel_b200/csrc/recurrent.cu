// Mechanisms that carry something from a request's last row to its next one, for mixers whose inputs
// come as one stacked product [rows, row_width] (a tensor or split-K partial sums).
//
//  token_shift       y[r] = h[r] + (h[r-1] - h[r]) * mu, channel by channel; the row before a request's
//                    first row of the step comes from its slot of a state table (zeros for a new request);
//                    `keep_last` then leaves the request's last h there.
//  conv_append       a short causal convolution over time on every channel of a query and a key
//                    projection (bias first, one filter a channel, no activation), the queries written
//                    out, the keys to the paged cache at each row's line; the last taps - 1 inputs of every
//                    channel live in a slot of a state table (`conv_history`).
//  decay_scan        a matrix memory S [d, e] a head with a decay a key channel and, optionally, the removal
//                    of what lies along a unit key:
//                        S <- diag(w) S - b (u^T S) + k v^T,   o = S^T r      (both first terms read the old S)
//                    Written on the old memory: with p = u^T S and q = (w r)^T S, o = q - p (b.r) + v (k.r),
//                    so both dot products of a row are reduced together. `gdelta_prep` (the generalized
//                    delta rule: decay through a small two-layer net, removal rate, unit keys) and
//                    `gate_prep` (tied gates: a forget gate with a lower bound, and one minus it as the input gate:
//                    w = f, k = 1 - f, no removal) make its inputs.
//  weighted_sum2     out = a * va + b * vb + vc with a weight a channel on each branch.
//
// Everything here is 32-bit; only the projections may come in bfloat16.
#include "common.cuh"

namespace kb {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float rc_sigmoid(float x) { return 1.f / (1.f + expf(-x)); }

// ------------------------------------------------------------------------------------------ token shift
template <typename T>
__global__ void token_shift_kernel(T* __restrict__ out, const T* __restrict__ h, const float* __restrict__ mu,
                                   const float* __restrict__ state, const int* __restrict__ row_entry,
                                   const int* __restrict__ entry_start, const int* __restrict__ slots, int entries, int n_slots,
                                   int width, int out_stride) {
    const int r = blockIdx.x;
    const int entry = row_entry[r];
    int r0 = r, slot = 0;
    if (entry >= 0 && entry < entries) {
        r0 = entry_start[entry];
        slot = slots[entry];
    }
    const bool kept = slot > 0 && slot < n_slots;
    for (int c = threadIdx.x; c < out_stride; c += blockDim.x) {
        float y = 0.f;
        if (c < width) {
            const float cur = Elem<T>::load(h + (size_t)r * width + c);
            const float before = r > r0 ? Elem<T>::load(h + (size_t)(r - 1) * width + c) : (kept ? state[(size_t)slot * width + c] : 0.f);
            y = fmaf(before - cur, mu[c], cur);
        }
        Elem<T>::store(out + (size_t)r * out_stride + c, y);
    }
}

template <typename T>
__global__ void keep_last_kernel(float* __restrict__ state, const T* __restrict__ h, const int* __restrict__ entry_start,
                                 const int* __restrict__ entry_end, const int* __restrict__ slots, int n_slots, int width) {
    const int entry = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int r0 = entry_start[entry], r1 = entry_end[entry];
    const int slot = slots[entry];
    if (c >= width || r1 <= r0 || slot <= 0 || slot >= n_slots) return;
    state[(size_t)slot * width + c] = Elem<T>::load(h + (size_t)(r1 - 1) * width + c);
}

// ------------------------------------------------------------------------------------------ convolutions ahead of attention
constexpr int CONV_MAX_TAPS = 16;

struct ConvParams {
    int row_width, q_off, k_off, nq, nk;      // columns of the stacked product; nq = hq d, nk = hkv d
    const float* bias;                        // [nq + nk] or null
    const float* conv;                        // [nq + nk, taps]: the last weight is the row's own
    float* state;                             // [slots, (taps - 1) (nq + nk)]
    const int* row_entry;
    const int* entry_start;
    const int* entry_end;
    const int* slots;
    const int* lines;
    int n_slots, entries, rows, taps, hkv, d, page_size, q_stride;
    long long table_lines;
};

template <typename TS, typename TO>
__global__ void conv_append_kernel(const Src<TS> src, const ConvParams p, TO* __restrict__ q_out, TO* __restrict__ k_table) {
    const int r = blockIdx.x;
    const int channels = p.nq + p.nk;
    const int entry = p.row_entry[r];
    int r0 = r, slot = 0;
    if (entry >= 0 && entry < p.entries) {
        r0 = p.entry_start[entry];
        slot = p.slots[entry];
    }
    const bool kept = slot > 0 && slot < p.n_slots;
    const float* hist = p.state + (size_t)(kept ? slot : 0) * (p.taps - 1) * channels;
    long long line = -1;
    if (k_table != nullptr) {
        line = p.lines[r];
        if (line >= p.table_lines) line = -1;
    }
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        const bool is_q = c < p.nq;
        if (!is_q && line < 0) continue;
        const int col = is_q ? p.q_off + c : p.k_off + (c - p.nq);
        const float b = p.bias != nullptr ? p.bias[c] : 0.f;
        float y = 0.f;
        for (int j = 0; j < p.taps; ++j) {                      // the input j rows back
            const int t = r - j;
            float x;
            if (t >= r0) x = src.at((size_t)t * p.row_width + col) + b;
            else if (kept) x = hist[(size_t)(p.taps - 1 + (t - r0)) * channels + c];
            else x = 0.f;
            y = fmaf(p.conv[(size_t)c * p.taps + (p.taps - 1 - j)], x, y);
        }
        if (is_q) {
            Elem<TO>::store(q_out + (size_t)r * p.q_stride + c, y);
        } else {
            const int ck = c - p.nq, h = ck / p.d, i = ck - h * p.d;
            Elem<TO>::store(k_table + kv_row(line, h, p.hkv, p.page_size) * p.d + i, y);
        }
    }
    for (int c = p.nq + threadIdx.x; c < p.q_stride; c += blockDim.x) Elem<TO>::store(q_out + (size_t)r * p.q_stride + c, 0.f);
}

// history <- the last taps - 1 inputs (bias added) of (history, this step's rows), per channel of a request.
template <typename TS>
__global__ void conv_history_kernel(const Src<TS> src, const ConvParams p) {
    const int entry = blockIdx.y;
    const int channels = p.nq + p.nk;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int r0 = p.entry_start[entry], r1 = p.entry_end[entry];
    const int slot = p.slots[entry];
    const int keep = p.taps - 1;
    if (r1 <= r0 || slot <= 0 || slot >= p.n_slots || keep <= 0) return;
    float* hist = p.state + (size_t)slot * keep * channels;
    const int col = c < p.nq ? p.q_off + c : p.k_off + (c - p.nq);
    const float b = p.bias != nullptr ? p.bias[c] : 0.f;
    const int n = r1 - r0;
    float fresh[CONV_MAX_TAPS];
#pragma unroll
    for (int i = 0; i < CONV_MAX_TAPS; ++i) {
        fresh[i] = 0.f;
        if (i < keep) {
            const int t = n - keep + i;
            fresh[i] = t >= 0 ? src.at((size_t)(r0 + t) * p.row_width + col) + b : hist[(size_t)(keep + t) * channels + c];
        }
    }
#pragma unroll
    for (int i = 0; i < CONV_MAX_TAPS; ++i)
        if (i < keep) hist[(size_t)i * channels + c] = fresh[i];
}

// ------------------------------------------------------------------------------------------ the scan's inputs
// Scratch of a step: vectors [rows, heads, NV, d] in the order (w r, w, k, u, b) (NV = 5 with the removal,
// else the first 3), values [rows, heads, e], scalars [rows, heads, 2] = (b.r, k.r).
struct ScanInputs {
    float* vec;
    float* val;
    float* scal;
    int nv;
};

struct GDeltaParams {
    int row_width, r_off, k_off, v_off, a_off, w1_off, lora;
    const float* w2;            // [lora, heads d]: the net's second layer turned, so that neighbouring threads read neighbouring weights
    const float* w0;            // [heads d]
    const float* a_bias;        // [heads d]
    float decay_scale;          // w = exp(-decay_scale * sigmoid(.))
    float unit_eps;
    int heads, d;
};

// One block RB rows. The small net's hidden layers tanh(w1 h) of the block's rows lie in shared memory; a thread a channel
// reads its weights of the second layer once for all RB rows and leaves the decay and the removal rate in the scratch
// (which the same block reads back below); a warp a (row, head) then makes the unit key and the two dot products.
// RB is 8 for prompt portions (the second layer's weights cross from L2 once in eight rows) and 1 for a few rows.
template <typename TS, int RB>
__global__ void __launch_bounds__(1024)
gdelta_prep_kernel(const Src<TS> src, const GDeltaParams p, const ScanInputs s, int rows) {
    extern __shared__ float hid[];                              // [RB][lora]
    const int r0 = blockIdx.x * RB;
    const int nr = min(RB, rows - r0);
    const int n = p.heads * p.d, d = p.d;
    for (int idx = threadIdx.x; idx < RB * p.lora; idx += blockDim.x) {
        const int rr = idx / p.lora, j = idx - rr * p.lora;
        hid[idx] = rr < nr ? tanhf(src.at((size_t)(r0 + rr) * p.row_width + p.w1_off + j)) : 0.f;
    }
    __syncthreads();
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
        float z[RB];
#pragma unroll
        for (int rr = 0; rr < RB; ++rr) z[rr] = 0.f;
        for (int j = 0; j < p.lora; ++j) {
            const float wj = p.w2[(size_t)j * n + c];
#pragma unroll
            for (int rr = 0; rr < RB; ++rr) z[rr] = fmaf(wj, hid[rr * p.lora + j], z[rr]);
        }
        const float w0 = p.w0[c], ab = p.a_bias[c];
        const int h = c / d, i = c - h * d;
#pragma unroll
        for (int rr = 0; rr < RB; ++rr) {
            if (rr < nr) {
                float* vec = s.vec + ((size_t)(r0 + rr) * p.heads + h) * 5 * d;
                vec[d + i] = expf(-p.decay_scale * rc_sigmoid(z[rr] + w0));
                vec[4 * d + i] = rc_sigmoid(src.at((size_t)(r0 + rr) * p.row_width + p.a_off + c) + ab);      // the rate; times the unit key below
            }
        }
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int pair = warp; pair < nr * p.heads; pair += warps) {
        const int rr = pair / p.heads, h = pair - rr * p.heads;
        const int r = r0 + rr;
        const size_t base = (size_t)r * p.row_width;
        float kk = 0.f;
        for (int i = lane; i < d; i += 32) {
            const float k = src.at(base + p.k_off + h * d + i);
            kk = fmaf(k, k, kk);
        }
        kk = warp_sum(kk);
        const float inv = 1.f / sqrtf(kk + p.unit_eps);
        float br = 0.f, kr = 0.f;
        float* vec = s.vec + ((size_t)r * p.heads + h) * 5 * d;
        for (int i = lane; i < d; i += 32) {
            const int c = h * d + i;
            const float k = src.at(base + p.k_off + c), q = src.at(base + p.r_off + c);
            const float u = k * inv, b = vec[4 * d + i] * u, w = vec[d + i];
            vec[i] = w * q;
            vec[2 * d + i] = k;
            vec[3 * d + i] = u;
            vec[4 * d + i] = b;
            br = fmaf(b, q, br);
            kr = fmaf(k, q, kr);
            s.val[(size_t)r * n + c] = src.at(base + p.v_off + c);
        }
        br = warp_sum(br);
        kr = warp_sum(kr);
        if (lane == 0) {
            s.scal[((size_t)r * p.heads + h) * 2] = br;
            s.scal[((size_t)r * p.heads + h) * 2 + 1] = kr;
        }
    }
}

struct GateParams {
    int row_width, q_off, f_off, v_off;
    const float* f_bias;        // [heads d]
    const float* lower;         // [heads d]
    int heads, d, e;
};

// One block a row: q = silu(.), f = l + (1 - l) sigmoid(. + bias); the scan's inputs are w r = f q, w = f, k = 1 - f.
template <typename TS>
__global__ void __launch_bounds__(256)
gate_prep_kernel(const Src<TS> src, const GateParams p, const ScanInputs s) {
    const int r = blockIdx.x;
    const size_t base = (size_t)r * p.row_width;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int h = warp; h < p.heads; h += warps) {
        float kr = 0.f;
        float* vec = s.vec + ((size_t)r * p.heads + h) * 3 * p.d;
        for (int i = lane; i < p.d; i += 32) {
            const int c = h * p.d + i;
            const float z = src.at(base + p.q_off + c);
            const float q = z * rc_sigmoid(z);
            const float l = p.lower[c];
            const float f = fmaf(1.f - l, rc_sigmoid(src.at(base + p.f_off + c) + p.f_bias[c]), l);
            vec[i] = f * q;
            vec[p.d + i] = f;
            vec[2 * p.d + i] = 1.f - f;
            kr = fmaf(1.f - f, q, kr);
        }
        kr = warp_sum(kr);
        if (lane == 0) {
            s.scal[((size_t)r * p.heads + h) * 2] = 0.f;
            s.scal[((size_t)r * p.heads + h) * 2 + 1] = kr;
        }
    }
    const int nv = p.heads * p.e;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) s.val[(size_t)r * nv + i] = src.at(base + p.v_off + i);
}

// ------------------------------------------------------------------------------------------ the scan
constexpr int SC = 4;                  // warps a block
constexpr int SCAN_R = 8;              // memory rows a lane can hold: d <= 32 * SCAN_R

struct ScanParams {
    const float* vec;           // [rows, heads, NV, d]
    const float* val;           // [rows, heads, e]
    const float* scal;          // [rows, heads, 2]
    float* state;               // [slots, heads, e, d]: a column of a head's memory lies together
    const int* entry_start;
    const int* entry_end;
    const int* slots;
    int n_slots, heads, d, e;
    float* out;                 // [rows, heads, e]
};

__device__ __forceinline__ void scan_copy4(float* dst, const float* src) {
    const uint32_t d32 = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d32), "l"(src) : "memory");
}
__device__ __forceinline__ void scan_copy16(float* dst, const float* src) {
    const uint32_t d32 = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d32), "l"(src) : "memory");
}

// R values that lie together, by the widest loads that fit (shared memory, 16-byte aligned where R >= 4).
template <int R>
__device__ __forceinline__ void scan_load(float (&dst)[R], const float* p) {
    if constexpr (R % 4 == 0) {
#pragma unroll
        for (int i = 0; i < R / 4; ++i) {
            const float4 v = reinterpret_cast<const float4*>(p)[i];
            dst[4 * i] = v.x; dst[4 * i + 1] = v.y; dst[4 * i + 2] = v.z; dst[4 * i + 3] = v.w;
        }
    } else if constexpr (R == 2) {
        const float2 v = *reinterpret_cast<const float2*>(p);
        dst[0] = v.x; dst[1] = v.y;
    } else {
#pragma unroll
        for (int i = 0; i < R; ++i) dst[i] = p[i];
    }
}

// One block = one request of the step x one head x SC * DW columns of the memory; a warp DW columns, lane l
// the rows R l .. R l + R - 1 of them in registers (a row's vectors then come from shared memory 16 bytes a load). R: rows a lane holds; CH: rows of the step staged at a time
// (asynchronous copies, the next chunk while this one is walked); REMOVAL: whether u and b exist.
template <int R, int CH, int DW, bool REMOVAL>
__global__ void __launch_bounds__(SC * 32)
decay_scan_kernel(const ScanParams p) {
    constexpr int NV = REMOVAL ? 5 : 3;
    constexpr int DP = R * 32;
    constexpr int COLS = SC * DW;
    constexpr int tail = NV * DP;                               // v [COLS] | b.r | k.r | padding
    constexpr int rowf = NV * DP + COLS + 4;
    extern __shared__ __align__(16) float staged[];             // [2][CH][rowf]
    const int entry = blockIdx.x, head = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int c0 = blockIdx.z * COLS + warp * DW;
    const int r0 = p.entry_start[entry], r1 = p.entry_end[entry];
    if (r1 <= r0) return;
    const int slot = p.slots[entry];
    const int d = p.d, e = p.e;
    if (slot <= 0 || slot >= p.n_slots) {                       // rows of no request: zeros, no state
        if (lane < DW && c0 + lane < e)
            for (int r = r0; r < r1; ++r) p.out[((size_t)r * p.heads + head) * e + c0 + lane] = 0.f;
        return;
    }
    float* st = p.state + ((size_t)slot * p.heads + head) * e * d;
    float S[DW][R];
#pragma unroll
    for (int ci = 0; ci < DW; ++ci)
#pragma unroll
        for (int i = 0; i < R; ++i) S[ci][i] = (c0 + ci < e && lane * R + i < d) ? st[(size_t)(c0 + ci) * d + lane * R + i] : 0.f;

    const bool wide = d % 4 == 0 && ((uintptr_t)p.vec & 15) == 0;
    auto stage = [&](int chunk, int buf) {
        const int rbase = r0 + chunk * CH;
        const int nr = min(CH, r1 - rbase);
        float* base = staged + (size_t)buf * CH * rowf;
        for (int t = warp; t < nr; t += SC) {
            float* row = base + (size_t)t * rowf;
            const float* vp = p.vec + ((size_t)(rbase + t) * p.heads + head) * NV * d;
#pragma unroll
            for (int v = 0; v < NV; ++v) {
                if (wide) {
                    for (int x = lane * 4; x < d; x += 128) scan_copy16(row + v * DP + x, vp + v * d + x);
                } else {
                    for (int x = lane; x < d; x += 32) scan_copy4(row + v * DP + x, vp + v * d + x);
                }
            }
        }
        for (int idx = tid; idx < nr * (COLS + 2); idx += SC * 32) {
            const int t = idx / (COLS + 2), x = idx - t * (COLS + 2);
            float* dst = base + (size_t)t * rowf + tail + x;
            const size_t r = (size_t)(rbase + t);
            if (x < COLS) {
                const int cc = blockIdx.z * COLS + x;
                if (cc < e) scan_copy4(dst, p.val + (r * p.heads + head) * e + cc);
                else *dst = 0.f;
            } else {
                scan_copy4(dst, p.scal + (r * p.heads + head) * 2 + (x - COLS));
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (d < DP) {                                               // the vectors' padding, once: no copy ever writes it
        const int pad = DP - d;
        for (int idx = tid; idx < 2 * CH * NV * pad; idx += SC * 32) {
            const int t = idx / (NV * pad), x = idx - t * NV * pad;
            const int v = x / pad, i = x - v * pad;
            staged[(size_t)t * rowf + v * DP + d + i] = 0.f;
        }
    }
    const bool hi16 = lane & 16;
    const int chunks = (r1 - r0 + CH - 1) / CH;
    stage(0, 0);
    for (int ch = 0; ch < chunks; ++ch) {
        if (ch + 1 < chunks) {
            stage(ch + 1, (ch + 1) & 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const int rbase = r0 + ch * CH;
        const int nr = min(CH, r1 - rbase);
        const float* rows = staged + (size_t)(ch & 1) * CH * rowf;
        for (int t = 0; t < nr; ++t) {
            const float* in = rows + (size_t)t * rowf;
            const float br = in[tail + COLS], kr = in[tail + COLS + 1];
            float wr[R], w[R], k[R], u[REMOVAL ? R : 1], b[REMOVAL ? R : 1];
            scan_load<R>(wr, in + lane * R);
            scan_load<R>(w, in + DP + lane * R);
            scan_load<R>(k, in + 2 * DP + lane * R);
            if constexpr (REMOVAL) {
                scan_load<R>(u, in + 3 * DP + lane * R);
                scan_load<R>(b, in + 4 * DP + lane * R);
            }
#pragma unroll
            for (int ci = 0; ci < DW; ++ci) {
                const float v = in[tail + warp * DW + ci];
                float o;
                if constexpr (REMOVAL) {
                    float xp = 0.f, xq = 0.f;
#pragma unroll
                    for (int i = 0; i < R; ++i) {
                        xp = fmaf(S[ci][i], u[i], xp);
                        xq = fmaf(S[ci][i], wr[i], xq);
                    }
                    // two sums over 32 lanes: the halves swap one of them, then both are reduced side by side (the lower lanes
                    // end with p, the upper with q). Two broadcasts then give every lane both; one exchange between the halves
                    // and a choice a lane instead measured a fifth slower (1.23 against 1.03 ms at 2,048 rows, 16 heads of 128).
                    float y = (hi16 ? xq : xp) + __shfl_xor_sync(0xffffffffu, hi16 ? xp : xq, 16);
                    y += __shfl_xor_sync(0xffffffffu, y, 8);
                    y += __shfl_xor_sync(0xffffffffu, y, 4);
                    y += __shfl_xor_sync(0xffffffffu, y, 2);
                    y += __shfl_xor_sync(0xffffffffu, y, 1);
                    const float pp = __shfl_sync(0xffffffffu, y, 0), qq = __shfl_sync(0xffffffffu, y, 16);
#pragma unroll
                    for (int i = 0; i < R; ++i) S[ci][i] = fmaf(k[i], v, fmaf(-b[i], pp, w[i] * S[ci][i]));
                    o = fmaf(v, kr, fmaf(-pp, br, qq));
                } else {
                    float xq = 0.f;
#pragma unroll
                    for (int i = 0; i < R; ++i) {
                        xq = fmaf(S[ci][i], wr[i], xq);
                        S[ci][i] = fmaf(k[i], v, w[i] * S[ci][i]);
                    }
                    xq = warp_sum(xq);
                    o = fmaf(v, kr, xq);
                }
                if (lane == 0 && c0 + ci < e) p.out[((size_t)(rbase + t) * p.heads + head) * e + c0 + ci] = o;
            }
        }
        __syncthreads();                                        // the chunk's buffer may be written again
    }
#pragma unroll
    for (int ci = 0; ci < DW; ++ci)
#pragma unroll
        for (int i = 0; i < R; ++i)
            if (c0 + ci < e && lane * R + i < d) st[(size_t)(c0 + ci) * d + lane * R + i] = S[ci][i];
}

// ------------------------------------------------------------------------------------------ two branches with a weight a channel
template <typename TA, typename TB>
__global__ void weighted_sum2_kernel(float* __restrict__ out, const Src<TA> a, const float* __restrict__ va, const Src<TB> b,
                                     const float* __restrict__ vb, const float* __restrict__ vc, long long total, int width, bool has_b) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int c = (int)(idx % width);
    float y = a.at((size_t)idx) * va[c];
    if (has_b) y = fmaf(b.at((size_t)idx), vb[c], y);
    if (vc != nullptr) y += vc[c];
    out[idx] = y;
}

}  // namespace kb

using namespace kb;

extern "C" int kb_token_shift(void* out, const void* h, int dt, const float* mu, float* state, const int* row_entry,
                              const int* entry_start, const int* entry_end, const int* slots, int entries, int n_slots, int rows,
                              int width, int out_stride, int keep, void* stream) {
    KB_REQUIRE(rows >= 0 && width > 0 && out_stride >= width && entries >= 0 && n_slots >= 1, "token_shift: rows %d, width %d (out %d), %d requests, %d slots",
               rows, width, out_stride, entries, n_slots);
    KB_REQUIRE(out && h && mu && state && row_entry && entry_start && entry_end && slots, "token_shift: a tensor is missing");
    KB_REQUIRE(entries <= 65535, "token_shift: too many requests for one launch");
    if (rows == 0 || entries == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = width >= 1024 ? 256 : 128;
    const dim3 kgrid((unsigned)((width + 127) / 128), entries);
    if (dt == KB_DT_F32) {
        token_shift_kernel<float><<<rows, threads, 0, s>>>((float*)out, (const float*)h, mu, state, row_entry, entry_start, slots, entries, n_slots, width, out_stride);
        if (int err = check_launch("token_shift")) return err;
        if (keep) keep_last_kernel<float><<<kgrid, 128, 0, s>>>(state, (const float*)h, entry_start, entry_end, slots, n_slots, width);
    } else if (dt == KB_DT_BF16) {
        token_shift_kernel<bf16><<<rows, threads, 0, s>>>((bf16*)out, (const bf16*)h, mu, state, row_entry, entry_start, slots, entries, n_slots, width, out_stride);
        if (int err = check_launch("token_shift")) return err;
        if (keep) keep_last_kernel<bf16><<<kgrid, 128, 0, s>>>(state, (const bf16*)h, entry_start, entry_end, slots, n_slots, width);
    } else {
        return fail("token_shift: dtype code %d is not known", dt);
    }
    return check_launch("token_shift keep");
}

extern "C" int kb_conv_append(void* q_out, int q_stride, void* k_table, int out_dt, const void* src, int in_dt, int splits,
                              long long split_stride, int row_width, int q_off, int k_off, const float* bias, const float* conv,
                              float* state, int n_slots, const int* row_entry, const int* entry_start, const int* entry_end,
                              const int* slots, const int* lines, int entries, int rows, int hq, int hkv, int d, int taps,
                              int write_kv, long long table_lines, int page_size, void* stream) {
    KB_REQUIRE(rows >= 0 && entries >= 0 && hq > 0 && hkv > 0 && d > 0, "conv_append: rows %d, heads %d / %d of %d", rows, hq, hkv, d);
    KB_REQUIRE(taps >= 1 && taps <= CONV_MAX_TAPS, "conv_append: a convolution of %d taps (1 to %d)", taps, CONV_MAX_TAPS);
    const int nq = hq * d, nk = hkv * d;
    KB_REQUIRE(row_width > 0 && q_off >= 0 && q_off + nq <= row_width && k_off >= 0 && k_off + nk <= row_width && q_stride >= nq,
               "conv_append: columns q %d, k %d do not fit a row of %d", q_off, k_off, row_width);
    KB_REQUIRE(splits >= 1 && (splits == 1 || split_stride >= (long long)rows * row_width), "conv_append: %d slices %lld apart", splits, split_stride);
    KB_REQUIRE(q_out && conv && state && n_slots >= 1 && row_entry && entry_start && entry_end && slots, "conv_append: a tensor is missing");
    KB_REQUIRE(!write_kv || (lines && k_table && table_lines > 0 && page_size > 0), "conv_append: no cache to write");
    KB_REQUIRE(entries <= 65535, "conv_append: too many requests for one launch");
    if (rows == 0 || entries == 0) return 0;
    ConvParams p;
    p.row_width = row_width; p.q_off = q_off; p.k_off = k_off; p.nq = nq; p.nk = nk; p.bias = bias; p.conv = conv; p.state = state;
    p.row_entry = row_entry; p.entry_start = entry_start; p.entry_end = entry_end; p.slots = slots; p.lines = lines;
    p.n_slots = n_slots; p.entries = entries; p.rows = rows; p.taps = taps; p.hkv = hkv; p.d = d; p.page_size = page_size;
    p.q_stride = q_stride; p.table_lines = table_lines;
    cudaStream_t s = (cudaStream_t)stream;
    void* kt = write_kv ? k_table : nullptr;
    const int channels = nq + nk;
    const int threads = channels >= 2048 ? 512 : 256;
#define KB_CONV(TS, TO)                                                                                                    \
    do {                                                                                                                   \
        conv_append_kernel<TS, TO><<<rows, threads, 0, s>>>(Src<TS>{(const TS*)src, splits, (size_t)split_stride}, p, (TO*)q_out, (TO*)kt); \
        if (int err = check_launch("conv_append")) return err;                                                             \
        if (taps > 1 && write_kv)                                                                                          \
            conv_history_kernel<TS><<<dim3((unsigned)((channels + 127) / 128), entries), 128, 0, s>>>(                      \
                Src<TS>{(const TS*)src, splits, (size_t)split_stride}, p);                                                 \
    } while (0)
    if (in_dt == KB_DT_F32 && out_dt == KB_DT_F32) KB_CONV(float, float);
    else if (in_dt == KB_DT_F32 && out_dt == KB_DT_BF16) KB_CONV(float, bf16);
    else if (in_dt == KB_DT_BF16 && out_dt == KB_DT_BF16) KB_CONV(bf16, bf16);
    else return fail("conv_append: dtype codes %d -> %d are not known", in_dt, out_dt);
#undef KB_CONV
    return check_launch("conv_append history");
}

// Floats of scratch for a step of `rows` rows of the scan: the vectors, the values, the two scalars.
extern "C" long long kb_decay_scan_scratch_floats(int rows, int heads, int d, int e, int removal) {
    return (long long)rows * heads * ((removal ? 5ll : 3ll) * d + e + 2);
}

// 0: the launcher chooses how many columns of the memory a warp of the scan holds; 1 or 2: that many (for tests and measurements).
static int g_scan_columns = 0;
extern "C" void kb_decay_scan_columns(int n) { g_scan_columns = (n == 1 || n == 2 || n == 4) ? n : 0; }

static int run_decay_scan(float* out, const ScanInputs& in, float* state, int n_slots, const int* entry_start, const int* entry_end,
                          const int* slots, int entries, int heads, int d, int e, bool removal, cudaStream_t s) {
    ScanParams p;
    p.vec = in.vec; p.val = in.val; p.scal = in.scal; p.state = state; p.entry_start = entry_start; p.entry_end = entry_end;
    p.slots = slots; p.n_slots = n_slots; p.heads = heads; p.d = d; p.e = e; p.out = out;
    int sms = 148;
    {
        int dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    }
    // columns a warp: the most that still leaves about four warps a multiprocessor (a warp reads a row's vectors once for all
    // its columns, and walks them as independent chains)
    const long long columns = (long long)entries * heads * e;
    int dw = g_scan_columns ? g_scan_columns : (columns / 4 >= 4ll * sms ? 4 : (columns / 2 >= 4ll * sms ? 2 : 1));
    KB_REQUIRE((e + SC * dw - 1) / (SC * dw) <= 65535 && heads <= 65535, "decay_scan: too many heads or value components for one launch");
    dim3 grid(entries, heads, (e + SC * dw - 1) / (SC * dw));
    const int need = (d + 31) / 32;
#define KB_SCAN(R, CH, W, REM)                                                                                    \
    do {                                                                                                          \
        const size_t smem = (size_t)2 * CH * ((REM ? 5 : 3) * R * 32 + SC * W + 4) * sizeof(float);               \
        if (smem > 48 * 1024) cudaFuncSetAttribute(decay_scan_kernel<R, CH, W, REM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        decay_scan_kernel<R, CH, W, REM><<<grid, SC * 32, smem, s>>>(p);                                          \
    } while (0)
#define KB_SCAN_W(R, CH)                                  \
    do {                                                  \
        if (removal) {                                    \
            if (dw == 4) KB_SCAN(R, CH, (R <= 4 ? 4 : 2), true);      \
            else if (dw == 2) KB_SCAN(R, CH, 2, true);    \
            else KB_SCAN(R, CH, 1, true);                 \
        } else {                                          \
            if (dw == 4) KB_SCAN(R, CH, (R <= 4 ? 4 : 2), false);     \
            else if (dw == 2) KB_SCAN(R, CH, 2, false);   \
            else KB_SCAN(R, CH, 1, false);                \
        }                                                 \
    } while (0)
    if (need <= 1) KB_SCAN_W(1, 16);
    else if (need <= 2) KB_SCAN_W(2, 16);
    else if (need <= 4) KB_SCAN_W(4, 8);
    else {                                                  // eight rows a lane: at most two columns a warp fit the registers
        if (dw == 4) {
            dw = 2;
            grid.z = (e + SC * dw - 1) / (SC * dw);
        }
        KB_SCAN_W(SCAN_R, 4);
    }
#undef KB_SCAN_W
#undef KB_SCAN
    return check_launch("decay_scan");
}

static int scan_common_checks(const char* what, const void* src, int splits, long long split_stride, int row_width, int rows, int entries,
                              int heads, int d, int e, const float* state, int n_slots, const void* a, const void* b, const void* c) {
    KB_REQUIRE(entries >= 0 && rows >= 0 && heads > 0 && d > 0 && e > 0, "%s: entries %d, rows %d, heads %d, sizes %d / %d", what, entries, rows, heads, d, e);
    KB_REQUIRE(d <= 32 * SCAN_R, "%s: a key size of %d is more than the kernel's %d", what, d, 32 * SCAN_R);
    KB_REQUIRE(splits >= 1 && (splits == 1 || split_stride >= (long long)rows * row_width), "%s: %d slices %lld apart", what, splits, split_stride);
    KB_REQUIRE(src && state && n_slots >= 1 && a && b && c, "%s: state, ranges or slots are missing", what);
    KB_REQUIRE(entries <= 65535, "%s: too many requests for one launch", what);
    return 0;
}

// The generalized delta rule's read-out [rows, heads, d] over the rows of a step.
extern "C" int kb_gdelta_scan(float* out, float* scratch, const void* src, int in_dt, int splits, long long split_stride, int row_width,
                              int r_off, int k_off, int v_off, int a_off, int w1_off, int lora, const float* w2, const float* w0,
                              const float* a_bias, float decay_scale, float unit_eps, float* state, int n_slots,
                              const int* entry_start, const int* entry_end, const int* slots, int entries, int rows, int heads, int d,
                              void* stream) {
    if (int err = scan_common_checks("gdelta", src, splits, split_stride, row_width, rows, entries, heads, d, d, state, n_slots, entry_start, entry_end, slots))
        return err;
    const long long n = (long long)heads * d;
    KB_REQUIRE(row_width > 0 && lora > 0 && r_off >= 0 && r_off + n <= row_width && k_off >= 0 && k_off + n <= row_width && v_off >= 0 &&
                   v_off + n <= row_width && a_off >= 0 && a_off + n <= row_width && w1_off >= 0 && w1_off + lora <= row_width,
               "gdelta: columns r %d, k %d, v %d, a %d, w1 %d (+%d) do not fit a row of %d", r_off, k_off, v_off, a_off, w1_off, lora, row_width);
    KB_REQUIRE(out && scratch && w2 && w0 && a_bias, "gdelta: weights or scratch are missing");
    const bool few = rows <= DEPENDENT_ROWS;
    const size_t smem = (size_t)(few ? 1 : 8) * lora * sizeof(float);
    KB_REQUIRE(smem <= 200 * 1024, "gdelta: a decay net of %d hidden values does not fit the shared memory of a block", lora);
    if (entries == 0 || rows == 0) return 0;
    GDeltaParams g;
    g.row_width = row_width; g.r_off = r_off; g.k_off = k_off; g.v_off = v_off; g.a_off = a_off; g.w1_off = w1_off; g.lora = lora;
    g.w2 = w2; g.w0 = w0; g.a_bias = a_bias; g.decay_scale = decay_scale; g.unit_eps = unit_eps; g.heads = heads; g.d = d;
    ScanInputs in;
    in.vec = scratch;
    in.val = in.vec + (size_t)rows * heads * 5 * d;
    in.scal = in.val + (size_t)rows * n;
    in.nv = 5;
    cudaStream_t s = (cudaStream_t)stream;
#define KB_GD(TS)                                                                                                          \
    do {                                                                                                                   \
        if (few) {                                                                                                         \
            if (smem > 48 * 1024) cudaFuncSetAttribute(gdelta_prep_kernel<TS, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            gdelta_prep_kernel<TS, 1><<<rows, 1024, smem, s>>>(Src<TS>{(const TS*)src, splits, (size_t)split_stride}, g, in, rows); /* few rows: a channel or two a thread */ \
        } else {                                                                                                           \
            if (smem > 48 * 1024) cudaFuncSetAttribute(gdelta_prep_kernel<TS, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            gdelta_prep_kernel<TS, 8><<<(rows + 7) / 8, 512, smem, s>>>(Src<TS>{(const TS*)src, splits, (size_t)split_stride}, g, in, rows); \
        }                                                                                                                  \
    } while (0)
    if (in_dt == KB_DT_F32) KB_GD(float);
    else if (in_dt == KB_DT_BF16) KB_GD(bf16);
    else return fail("gdelta: dtype code %d is not known", in_dt);
#undef KB_GD
    if (int err = check_launch("gdelta prep")) return err;
    return run_decay_scan(out, in, state, n_slots, entry_start, entry_end, slots, entries, heads, d, d, true, s);
}

// The read-out [rows, heads, e] of the memory behind a forget gate with a lower bound.
extern "C" int kb_gate_scan(float* out, float* scratch, const void* src, int in_dt, int splits, long long split_stride, int row_width,
                            int q_off, int f_off, int v_off, const float* f_bias, const float* lower, float* state, int n_slots,
                            const int* entry_start, const int* entry_end, const int* slots, int entries, int rows, int heads, int d,
                            int e, void* stream) {
    if (int err = scan_common_checks("gate_scan", src, splits, split_stride, row_width, rows, entries, heads, d, e, state, n_slots, entry_start, entry_end, slots))
        return err;
    const long long nq = (long long)heads * d, nv = (long long)heads * e;
    KB_REQUIRE(row_width > 0 && q_off >= 0 && q_off + nq <= row_width && f_off >= 0 && f_off + nq <= row_width && v_off >= 0 && v_off + nv <= row_width,
               "gate_scan: columns q %d, f %d, v %d do not fit a row of %d", q_off, f_off, v_off, row_width);
    KB_REQUIRE(out && scratch && f_bias && lower, "gate_scan: weights or scratch are missing");
    if (entries == 0 || rows == 0) return 0;
    GateParams g;
    g.row_width = row_width; g.q_off = q_off; g.f_off = f_off; g.v_off = v_off; g.f_bias = f_bias; g.lower = lower;
    g.heads = heads; g.d = d; g.e = e;
    ScanInputs in;
    in.vec = scratch;
    in.val = in.vec + (size_t)rows * heads * 3 * d;
    in.scal = in.val + (size_t)rows * nv;
    in.nv = 3;
    cudaStream_t s = (cudaStream_t)stream;
    if (in_dt == KB_DT_F32) gate_prep_kernel<float><<<rows, 256, 0, s>>>(Src<float>{(const float*)src, splits, (size_t)split_stride}, g, in);
    else if (in_dt == KB_DT_BF16) gate_prep_kernel<bf16><<<rows, 256, 0, s>>>(Src<bf16>{(const bf16*)src, splits, (size_t)split_stride}, g, in);
    else return fail("gate_scan: dtype code %d is not known", in_dt);
    if (int err = check_launch("gate_scan prep")) return err;
    return run_decay_scan(out, in, state, n_slots, entry_start, entry_end, slots, entries, heads, d, e, false, s);
}

extern "C" int kb_weighted_sum2(float* out, const void* a, int a_dt, int a_splits, long long a_stride, const float* va, const void* b,
                                int b_dt, int b_splits, long long b_stride, const float* vb, const float* vc, long long rows, int width,
                                void* stream) {
    KB_REQUIRE(rows >= 0 && width > 0 && out && a && va, "weighted_sum2: rows %lld, width %d", rows, width);
    KB_REQUIRE(b == nullptr || vb != nullptr, "weighted_sum2: a second branch without its weights");
    KB_REQUIRE(a_splits >= 1 && b_splits >= 1, "weighted_sum2: %d / %d slices", a_splits, b_splits);
    if (rows == 0) return 0;
    const long long total = rows * width;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    const bool has_b = b != nullptr;
    const void* bp = has_b ? b : a;
    if (!has_b) { b_dt = a_dt; b_splits = 1; b_stride = 0; }
#define KB_WS(TA, TB)                                                                                                       \
    weighted_sum2_kernel<TA, TB><<<blocks, 256, 0, s>>>(out, Src<TA>{(const TA*)a, a_splits, (size_t)a_stride}, va,           \
                                                       Src<TB>{(const TB*)bp, b_splits, (size_t)b_stride}, vb, vc, total, width, has_b)
    if (a_dt == KB_DT_F32 && b_dt == KB_DT_F32) KB_WS(float, float);
    else if (a_dt == KB_DT_F32 && b_dt == KB_DT_BF16) KB_WS(float, bf16);
    else if (a_dt == KB_DT_BF16 && b_dt == KB_DT_F32) KB_WS(bf16, float);
    else if (a_dt == KB_DT_BF16 && b_dt == KB_DT_BF16) KB_WS(bf16, bf16);
    else return fail("weighted_sum2: dtype codes %d, %d are not known", a_dt, b_dt);
#undef KB_WS
    return check_launch("weighted_sum2");
}
