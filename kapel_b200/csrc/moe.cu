// A mixture of experts: the router, the lists of tokens by expert, the experts' two products as
// grouped products over those lists, and the weighted sum.
//
//  route     z = router . h in 32-bit; s = sigmoid(z) (or softmax over the experts; or z itself, the
//            chosen experts then weighted by the softmax over the chosen logits alone); choice scores
//            s + correction; experts in equal groups of neighbours, a group's score the sum of its
//            `group_top` largest choice scores, only the best `keep_groups` groups stay eligible;
//            the `top` largest eligible choice scores are chosen (the lower number wins a tie) and
//            weighted by s, optionally divided by their sum.
//  sort      (token, k) pairs listed by expert, and the row tiles of the grouped products.
//  product   out[pair] = act(A[row of pair] . W[expert of pair]^T): a block a (row tile of one
//            expert, column tile); bfloat16 by mma.sync with 32-bit sums, float32 by FMA in
//            ascending k. What a pair's row computes does not depend on its place in a tile.
//  combine   out[token] = sum over k, in order, of weight[token, k] * y[token * top + k].
#include "common.cuh"

namespace kb {

typedef __nv_bfloat16 bf16;

// ------------------------------------------------------------------------------------------ route
constexpr int ROUTE_THREADS = 256;

template <typename TH>
__global__ void __launch_bounds__(ROUTE_THREADS)
moe_route_kernel(const TH* __restrict__ h, const float* __restrict__ router, const float* __restrict__ correction,
                 int* __restrict__ experts_out, float* __restrict__ weights_out, int width, int n_experts, int top, int groups,
                 int keep_groups, int group_top, int softmax, int renormalize) {
    extern __shared__ float sm[];
    float* score = sm;                         // [E] s
    float* choice = sm + n_experts;            // [E] s + correction
    float* gscore = choice + n_experts;        // [groups]
    int* state = reinterpret_cast<int*>(gscore + groups);   // [E] 0 eligible, 1 its group was dropped, 2 chosen
    const int r = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const TH* hr = h + (size_t)r * width;
    for (int x = warp; x < n_experts; x += ROUTE_THREADS / 32) {
        const float* w = router + (size_t)x * width;
        // eight loads of each operand ahead of their eight additions, which keep the order of i
        float acc = 0.f;
        for (int i0 = lane; i0 < width; i0 += 32 * 8) {
            float hv[8], wv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = i0 + 32 * u;
                hv[u] = i < width ? Elem<TH>::load(hr + i) : 0.f;
                wv[u] = i < width ? w[i] : 0.f;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) acc = fmaf(hv[u], wv[u], acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) score[x] = acc;
    }
    __syncthreads();
    if (threadIdx.x != 0) return;
    if (softmax == 2) {
        // the logits themselves choose; the chosen ones are weighted below
    } else if (softmax) {
        float mx = -INFINITY;
        for (int x = 0; x < n_experts; ++x) mx = fmaxf(mx, score[x]);
        float total = 0.f;
        for (int x = 0; x < n_experts; ++x) { score[x] = expf(score[x] - mx); total += score[x]; }
        for (int x = 0; x < n_experts; ++x) score[x] /= total;
    } else {
        for (int x = 0; x < n_experts; ++x) score[x] = 1.f / (1.f + expf(-score[x]));
    }
    for (int x = 0; x < n_experts; ++x) {
        choice[x] = score[x] + (correction ? correction[x] : 0.f);
        state[x] = 0;
    }
    const int per = n_experts / groups;
    if (groups > 1 && keep_groups < groups) {
        for (int g = 0; g < groups; ++g) {
            // the sum of the group's `group_top` largest choice scores, by repeated selection
            float total = 0.f;
            int taken[8];
            const int want = min(min(group_top, per), 8);
            for (int t = 0; t < want; ++t) {
                int best = -1;
                float bv = -INFINITY;
                for (int x = 0; x < per; ++x) {
                    bool used = false;
                    for (int u = 0; u < t; ++u) used |= taken[u] == x;
                    if (used) continue;
                    const float v = choice[g * per + x];
                    if (best < 0 || v > bv) { best = x; bv = v; }
                }
                taken[t] = best;
                total += bv;
            }
            gscore[g] = total;
        }
        // all but the best `keep_groups` groups lose their experts
        for (int drop = 0; drop < groups - keep_groups; ++drop) {
            int worst = -1;
            float wv = INFINITY;
            for (int g = groups - 1; g >= 0; --g) {          // among equals the higher number goes first
                const float v = gscore[g];
                if (v == INFINITY) continue;                 // already dropped
                if (worst < 0 || v < wv) { worst = g; wv = v; }
            }
            if (worst < 0) break;
            gscore[worst] = INFINITY;
            for (int x = 0; x < per; ++x) state[worst * per + x] = 1;
        }
    }
    float total = 0.f;
    for (int t = 0; t < top; ++t) {
        int best = -1;
        float bv = -INFINITY;
        for (int x = 0; x < n_experts; ++x) {
            if (state[x] != 0) continue;
            if (best < 0 || choice[x] > bv) { best = x; bv = choice[x]; }
        }
        if (best < 0)                                        // cannot happen with the sizes checked; stay in range all the same
            for (int x = 0; x < n_experts && best < 0; ++x)
                if (state[x] != 2) best = x;
        if (best < 0) best = 0;
        experts_out[(size_t)r * top + t] = best;
        weights_out[(size_t)r * top + t] = score[best];
        total += score[best];
        state[best] = 2;
    }
    if (softmax == 2) {                                      // softmax over the chosen logits alone (the first chosen is the largest)
        float* w = weights_out + (size_t)r * top;
        const float mx = w[0];
        float sum = 0.f;
        for (int t = 0; t < top; ++t) { w[t] = expf(w[t] - mx); sum += w[t]; }
        for (int t = 0; t < top; ++t) w[t] /= sum;
        return;
    }
    if (renormalize && total > 0.f)
        for (int t = 0; t < top; ++t) weights_out[(size_t)r * top + t] /= total;
}

// ------------------------------------------------------------------------------------------- sort
constexpr int GM = 32;         // rows of a grouped product's tile: few rows an expert, and the 32-bit path
constexpr int GM_LARGE = 64;   // and where an expert has many rows (bfloat16)
constexpr int SORT_THREADS = 1024;

// One block. offsets [E + 1]; order [pairs]: pair numbers by expert (any order within an expert);
// tile_expert / tile_first / tile_rows [tile_cap] and n_tiles[0].
__global__ void __launch_bounds__(SORT_THREADS)
moe_sort_kernel(const int* __restrict__ experts, int pairs, int n_experts, int* __restrict__ offsets, int* __restrict__ order,
                int* __restrict__ tile_expert, int* __restrict__ tile_first, int* __restrict__ tile_rows, int* __restrict__ n_tiles,
                int tile_cap, int rows_a_tile) {
    extern __shared__ int si[];
    int* count = si;                 // [E]
    int* cursor = si + n_experts;    // [E]
    for (int x = threadIdx.x; x < n_experts; x += blockDim.x) count[x] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int x = experts[i];
        if (x >= 0 && x < n_experts) atomicAdd(&count[x], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tiles = 0;
        for (int x = 0; x < n_experts; ++x) {
            offsets[x] = at;
            cursor[x] = at;
            for (int t = 0; t < count[x]; t += rows_a_tile) {
                if (tiles < tile_cap) {
                    tile_expert[tiles] = x;
                    tile_first[tiles] = at + t;
                    tile_rows[tiles] = min(rows_a_tile, count[x] - t);
                }
                ++tiles;
            }
            at += count[x];
        }
        offsets[n_experts] = at;
        n_tiles[0] = min(tiles, tile_cap);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int x = experts[i];
        if (x >= 0 && x < n_experts) order[atomicAdd(&cursor[x], 1)] = i;
    }
}

// ---------------------------------------------------------------------------------------- product
constexpr int GN = 64;         // columns of a tile
constexpr int GK = 32;         // k step
constexpr int GEMM_THREADS = 128;

__device__ __forceinline__ float moe_act(float v, int act) {
    if (act == 1) { const float r = fmaxf(v, 0.f); return r * r; }     // the square of relu
    if (act == 2) return gelu_tanh(v);
    if (act == 3) return silu(v);
    return v;
}

struct GroupedParams {
    const void* a;             // [*, k]: rows taken through `a_row`
    const void* w;             // [experts, n, k]
    void* out;                 // [pairs, n]: rows placed through `out_row`
    const int* order;          // [pairs]: the pair at each sorted place
    const int* tile_expert;
    const int* tile_first;
    const int* tile_rows;
    const int* n_tiles;
    int n, k, top, act;
    int a_by;                  // 0: A's row is the sorted place; 1: the pair's token (pair / top)
    int out_by;                // 0: the output row is the sorted place; 1: the pair number
};

// float32: each thread 4 rows x 4 columns, k ascending.
__global__ void __launch_bounds__(GEMM_THREADS)
moe_grouped_f32_kernel(const GroupedParams p) {
    const int tile = blockIdx.x;
    if (tile >= p.n_tiles[0]) return;
    __shared__ float As[GK][GM + 1];
    __shared__ float Ws[GK][GN + 1];
    __shared__ int arow[GM], orow[GM];
    const int expert = p.tile_expert[tile], first = p.tile_first[tile], nrows = p.tile_rows[tile];
    const int n0 = blockIdx.y * GN;
    const int tid = threadIdx.x;
    if (tid < GM) {
        const int place = first + min(tid, nrows - 1);
        const int pair = p.order[place];
        arow[tid] = p.a_by ? pair / p.top : place;
        orow[tid] = p.out_by ? pair : place;
    }
    __syncthreads();
    const float* A = static_cast<const float*>(p.a);
    const float* W = static_cast<const float*>(p.w) + (size_t)expert * p.n * p.k;
    const int tr = (tid / 16) * 4, tc = (tid % 16) * 4;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < p.k; k0 += GK) {
        for (int i = tid; i < GM * GK; i += GEMM_THREADS) {
            const int row = i / GK, kk = i % GK;
            As[kk][row] = (k0 + kk < p.k) ? A[(size_t)arow[row] * p.k + k0 + kk] : 0.f;
        }
        for (int i = tid; i < GN * GK; i += GEMM_THREADS) {
            const int col = i / GK, kk = i % GK;
            Ws[kk][col] = (n0 + col < p.n && k0 + kk < p.k) ? W[(size_t)(n0 + col) * p.k + k0 + kk] : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < GK; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][tr + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tc + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
    float* out = static_cast<float*>(p.out);
    for (int i = 0; i < 4; ++i) {
        if (tr + i >= nrows) continue;
        for (int j = 0; j < 4; ++j)
            if (n0 + tc + j < p.n) out[(size_t)orow[tr + i] * p.n + n0 + tc + j] = moe_act(acc[i][j], p.act);
    }
}

// bfloat16 operands, 32-bit sums by mma.sync m16n8k16. A block takes TM rows of one expert by TN
// columns with WM x WN warps; tiles of TK k values arrive by 16-byte asynchronous copies, three
// stages deep, so that a block that walks one expert's weights for a handful of rows (a decoding
// step) keeps loads in flight instead of waiting for each tile; rows of k that are no multiple of
// 8 are loaded value by value. Two shapes: 32 x 64 (few rows an expert) and 64 x 128 (prompts); 128 x 128 was
// built and measured no faster (the products run at about 215 TFLOP/s either way).
constexpr int BSTAGES = 3;

__device__ __forceinline__ void moe_copy16(void* dst, const void* src, bool valid) {
    const uint32_t d32 = (uint32_t)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;                        // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d32), "l"(src), "r"(bytes) : "memory");
}

__device__ __forceinline__ void moe_ldmatrix4(uint32_t (&r)[4], const void* at) {
    const uint32_t a32 = (uint32_t)__cvta_generic_to_shared(at);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a32));
}

template <typename TO, int TM, int TN, int WM, int WN, int TK>
__global__ void __launch_bounds__(WM * WN * 32)
moe_grouped_bf16_kernel(const GroupedParams p) {
    static_assert((TN / WN / 8) % 2 == 0, "a warp's n8 tiles come in pairs");
    constexpr int THREADS = WM * WN * 32;
    constexpr int MT = TM / WM / 16, NT = TN / WN / 8;       // m16 and n8 tiles a warp
    const int tile = blockIdx.x;
    if (tile >= p.n_tiles[0]) return;
    extern __shared__ __align__(16) unsigned char moe_smem[];      // As [stages][TM][TK + 8] | Ws [stages][TN][TK + 8] | arow | orow
    bf16 (*As)[TM][TK + 8] = reinterpret_cast<bf16 (*)[TM][TK + 8]>(moe_smem);
    bf16 (*Ws)[TN][TK + 8] = reinterpret_cast<bf16 (*)[TN][TK + 8]>(moe_smem + sizeof(bf16) * BSTAGES * TM * (TK + 8));
    int* arow = reinterpret_cast<int*>(moe_smem + sizeof(bf16) * BSTAGES * (TM + TN) * (TK + 8));
    int* orow = arow + TM;
    const int expert = p.tile_expert[tile], first = p.tile_first[tile], nrows = p.tile_rows[tile];
    const int n0 = blockIdx.y * TN;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wm = warp / WN, wn = warp % WN;
    if (tid < TM) {
        const int place = first + min(tid, nrows - 1);
        const int pair = p.order[place];
        arow[tid] = p.a_by ? pair / p.top : place;
        orow[tid] = p.out_by ? pair : place;
    }
    __syncthreads();
    const bf16* A = static_cast<const bf16*>(p.a);
    const bf16* W = static_cast<const bf16*>(p.w) + (size_t)expert * p.n * p.k;
    const bool vec = (p.k % 8) == 0 && ((((uintptr_t)A) | ((uintptr_t)W)) & 15) == 0;
    const int nk = (p.k + TK - 1) / TK;
    auto load_stage = [&](int kt, int st) {
        const int k0 = kt * TK;
        if (vec) {
            for (int i = tid; i < TM * (TK / 8); i += THREADS) {
                const int row = i / (TK / 8), kk = (i % (TK / 8)) * 8;
                const bool ok = k0 + kk < p.k;
                moe_copy16(&As[st][row][kk], A + (size_t)arow[row] * p.k + (ok ? k0 + kk : 0), ok);
            }
            for (int i = tid; i < TN * (TK / 8); i += THREADS) {
                const int col = i / (TK / 8), kk = (i % (TK / 8)) * 8;
                const bool ok = n0 + col < p.n && k0 + kk < p.k;
                moe_copy16(&Ws[st][col][kk], W + (ok ? (size_t)(n0 + col) * p.k + k0 + kk : 0), ok);
            }
        } else {
            for (int i = tid; i < TM * TK; i += THREADS) {
                const int row = i / TK, kk = i % TK;
                As[st][row][kk] = (k0 + kk < p.k) ? A[(size_t)arow[row] * p.k + k0 + kk] : __float2bfloat16_rn(0.f);
            }
            for (int i = tid; i < TN * TK; i += THREADS) {
                const int col = i / TK, kk = i % TK;
                Ws[st][col][kk] = (n0 + col < p.n && k0 + kk < p.k) ? W[(size_t)(n0 + col) * p.k + k0 + kk] : __float2bfloat16_rn(0.f);
            }
        }
    };
    float acc[MT][NT][4] = {};
    const int grp = lane >> 2, qd = lane & 3;
#pragma unroll
    for (int st = 0; st < BSTAGES - 1; ++st) {
        if (st < nk) load_stage(st, st);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int kt = 0; kt < nk; ++kt) {
        asm volatile("cp.async.wait_group %0;" ::"n"(BSTAGES - 2) : "memory");
        __syncthreads();                                      // tile kt has landed; everyone is done with tile kt - 1
        if (kt + BSTAGES - 1 < nk) load_stage(kt + BSTAGES - 1, (kt + BSTAGES - 1) % BSTAGES);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const int st = kt % BSTAGES;
#pragma unroll
        for (int ks = 0; ks < TK; ks += 16) {
            // four 8 x 8 pieces an instruction: an m16 x k16 piece of A, or the k16 pieces of two n8 tiles of W
            uint32_t af[MT][4], bfr[NT][2];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
                moe_ldmatrix4(af[mt], &As[st][wm * (TM / WM) + mt * 16 + (lane & 15)][ks + (lane >> 4) * 8]);
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
                uint32_t b4[4];
                moe_ldmatrix4(b4, &Ws[st][wn * (TN / WN) + np * 16 + (lane & 7) + ((lane >> 4) << 3)][ks + ((lane >> 3) & 1) * 8]);
                bfr[2 * np][0] = b4[0]; bfr[2 * np][1] = b4[1];
                bfr[2 * np + 1][0] = b4[2]; bfr[2 * np + 1][1] = b4[3];
            }
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
                    asm volatile(
                        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                        : "+f"(acc[mt][nt][0]), "+f"(acc[mt][nt][1]), "+f"(acc[mt][nt][2]), "+f"(acc[mt][nt][3])
                        : "r"(af[mt][0]), "r"(af[mt][1]), "r"(af[mt][2]), "r"(af[mt][3]), "r"(bfr[nt][0]), "r"(bfr[nt][1]));
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    TO* out = static_cast<TO*>(p.out);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const int row = wm * (TM / WM) + mt * 16 + grp + (v >= 2 ? 8 : 0);
                const int col = n0 + wn * (TN / WN) + nt * 8 + qd * 2 + (v & 1);
                if (row < nrows && col < p.n) Elem<TO>::store(out + (size_t)orow[row] * p.n + col, moe_act(acc[mt][nt][v], p.act));
            }
}

// ---------------------------------------------------------------------------------------- combine
// `also` (a tensor or split-K partial sums of the output's shape, or none) is added behind the experts' sum: an
// expert that every token uses.
template <typename TO, typename TA>
__global__ void moe_combine_kernel(TO* __restrict__ out, const float* __restrict__ y, const float* __restrict__ weights,
                                   long long rows, int width, int top, const Src<TA> also) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * width) return;
    const long long r = i / width;
    const int c = (int)(i - r * width);
    float acc = 0.f;
    for (int t = 0; t < top; ++t) acc = fmaf(weights[r * top + t], y[((size_t)r * top + t) * width + c], acc);
    if (also.p != nullptr) acc += also.at((size_t)i);
    Elem<TO>::store(out + i, acc);
}

}  // namespace kb

using namespace kb;

// Rows of a grouped product's tile when an expert has about `rows_an_expert` rows.
extern "C" int kb_moe_tile_rows(int dt, long long rows_an_expert) {
    return (dt == KB_DT_BF16 && rows_an_expert >= 48) ? GM_LARGE : GM;
}

extern "C" int kb_moe_route(int* experts, float* weights, const void* h, int h_dt, const float* router, const float* correction,
                            int rows, int width, int n_experts, int top, int groups, int keep_groups, int group_top,
                            int softmax, int renormalize, void* stream) {
    KB_REQUIRE(softmax >= 0 && softmax <= 2, "moe_route: scoring code %d is not known (0 sigmoid, 1 softmax, 2 softmax over the chosen)", softmax);
    KB_REQUIRE(rows >= 0 && width > 0 && n_experts > 0 && top > 0 && top <= n_experts, "moe_route: rows %d, width %d, %d experts, top %d", rows, width, n_experts, top);
    KB_REQUIRE(groups >= 1 && n_experts % groups == 0 && keep_groups >= 1 && keep_groups <= groups,
               "moe_route: %d experts in %d groups of which %d are kept", n_experts, groups, keep_groups);
    KB_REQUIRE(keep_groups * (n_experts / groups) >= top, "moe_route: %d groups of %d experts cannot give %d", keep_groups, n_experts / groups, top);
    KB_REQUIRE(group_top >= 1 && group_top <= 8, "moe_route: a group's score adds up %d scores (1 to 8)", group_top);
    const size_t smem = ((size_t)3 * n_experts + groups) * sizeof(float);
    KB_REQUIRE(smem <= 48 * 1024, "moe_route: %d experts are too many for the router's shared memory", n_experts);
    if (rows == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (h_dt == KB_DT_F32)
        moe_route_kernel<float><<<rows, ROUTE_THREADS, smem, s>>>((const float*)h, router, correction, experts, weights, width, n_experts, top,
                                                                  groups, keep_groups, group_top, softmax, renormalize);
    else if (h_dt == KB_DT_BF16)
        moe_route_kernel<bf16><<<rows, ROUTE_THREADS, smem, s>>>((const bf16*)h, router, correction, experts, weights, width, n_experts, top,
                                                                 groups, keep_groups, group_top, softmax, renormalize);
    else return fail("moe_route: dtype code %d is not known", h_dt);
    return check_launch("moe_route");
}

extern "C" int kb_moe_sort(const int* experts, int pairs, int n_experts, int* offsets, int* order, int* tile_expert,
                           int* tile_first, int* tile_rows, int* n_tiles, int tile_cap, int rows_a_tile, void* stream) {
    KB_REQUIRE(pairs >= 0 && n_experts > 0 && tile_cap >= 0, "moe_sort: %d pairs, %d experts", pairs, n_experts);
    KB_REQUIRE(rows_a_tile == GM || rows_a_tile == GM_LARGE, "moe_sort: tiles of %d rows (%d or %d)", rows_a_tile, GM, GM_LARGE);
    const size_t smem = (size_t)2 * n_experts * sizeof(int);
    KB_REQUIRE(smem <= 48 * 1024, "moe_sort: %d experts are too many", n_experts);
    moe_sort_kernel<<<1, SORT_THREADS, smem, (cudaStream_t)stream>>>(experts, pairs, n_experts, offsets, order, tile_expert, tile_first,
                                                                    tile_rows, n_tiles, tile_cap, rows_a_tile);
    return check_launch("moe_sort");
}

// act: 0 none, 1 relu squared, 2 gelu_tanh, 3 silu.
extern "C" int kb_moe_grouped(void* out, int out_dt, const void* a, const void* w, int dt, const int* order, const int* tile_expert,
                              const int* tile_first, const int* tile_rows, const int* n_tiles, int tile_cap, int rows_a_tile, int n,
                              int k, int top, int act, int a_by_token, int out_by_pair, void* stream) {
    KB_REQUIRE(n > 0 && k > 0 && top > 0 && tile_cap >= 0, "moe_grouped: n %d, k %d, top %d", n, k, top);
    KB_REQUIRE(rows_a_tile == GM || (rows_a_tile == GM_LARGE && dt == KB_DT_BF16), "moe_grouped: tiles of %d rows", rows_a_tile);
    KB_REQUIRE(act >= 0 && act <= 3, "moe_grouped: activation code %d is not known", act);
    if (tile_cap == 0) return 0;
    GroupedParams p;
    p.a = a; p.w = w; p.out = out; p.order = order; p.tile_expert = tile_expert; p.tile_first = tile_first; p.tile_rows = tile_rows;
    p.n_tiles = n_tiles; p.n = n; p.k = k; p.top = top; p.act = act; p.a_by = a_by_token; p.out_by = out_by_pair;
    const int tn = rows_a_tile == GM ? GN : 128;
    const int col_tiles = (n + tn - 1) / tn;
    KB_REQUIRE(col_tiles <= 65535, "moe_grouped: %d columns are too many for one launch", n);
    dim3 grid(tile_cap, col_tiles);
    cudaStream_t s = (cudaStream_t)stream;
    if (dt == KB_DT_F32) {
        KB_REQUIRE(out_dt == KB_DT_F32, "moe_grouped: a 32-bit product writes 32-bit");
        moe_grouped_f32_kernel<<<grid, GEMM_THREADS, 0, s>>>(p);
    } else if (dt == KB_DT_BF16) {
        KB_REQUIRE(out_dt == KB_DT_F32 || out_dt == KB_DT_BF16, "moe_grouped: output dtype code %d is not known", out_dt);
#define KB_MOE_TILE(TO, TM, TN, WM, WN, TK)                                                                                \
    do {                                                                                                                   \
        constexpr size_t bytes = sizeof(bf16) * BSTAGES * (TM + TN) * (TK + 8) + 2 * TM * sizeof(int);                     \
        if (bytes > 48 * 1024) {                                                                                           \
            static bool set = false;                                                                                       \
            if (!set) {                                                                                                    \
                if (cudaFuncSetAttribute(moe_grouped_bf16_kernel<TO, TM, TN, WM, WN, TK>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                         (int)bytes) != cudaSuccess)                                                       \
                    return fail("moe_grouped: cannot have %zu bytes of shared memory", bytes);                             \
                set = true;                                                                                                \
            }                                                                                                              \
        }                                                                                                                  \
        moe_grouped_bf16_kernel<TO, TM, TN, WM, WN, TK><<<grid, WM * WN * 32, bytes, s>>>(p);                                \
    } while (0)
        if (rows_a_tile == GM_LARGE) {
            if (out_dt == KB_DT_F32) KB_MOE_TILE(float, GM_LARGE, 128, 2, 4, 32);
            else KB_MOE_TILE(bf16, GM_LARGE, 128, 2, 4, 32);
        } else {
            if (out_dt == KB_DT_F32) KB_MOE_TILE(float, GM, GN, 1, 4, 64);
            else KB_MOE_TILE(bf16, GM, GN, 1, 4, 64);
        }
#undef KB_MOE_TILE
    } else return fail("moe_grouped: dtype code %d is not known", dt);
    return check_launch("moe_grouped");
}

extern "C" int kb_moe_combine(void* out, int out_dt, const float* y, const float* weights, long long rows, int width, int top,
                              const void* also, int also_dt, int also_splits, long long also_stride, void* stream) {
    KB_REQUIRE(rows >= 0 && width > 0 && top > 0, "moe_combine: rows %lld, width %d, top %d", rows, width, top);
    KB_REQUIRE(also == nullptr || also_splits >= 1, "moe_combine: an addend of %d slices", also_splits);
    if (rows == 0) return 0;
    const long long blocks = (rows * width + 255) / 256;
    KB_REQUIRE(blocks <= 0x7fffffffll, "moe_combine: too many rows for one launch");
    cudaStream_t s = (cudaStream_t)stream;
#define KB_COMBINE(TO, TA) \
    moe_combine_kernel<TO, TA><<<(unsigned)blocks, 256, 0, s>>>((TO*)out, y, weights, rows, width, top, Src<TA>{(const TA*)also, also ? also_splits : 1, (size_t)also_stride})
    const bool narrow = also != nullptr && also_dt == KB_DT_BF16;
    KB_REQUIRE(also == nullptr || also_dt == KB_DT_F32 || also_dt == KB_DT_BF16, "moe_combine: addend dtype code %d is not known", also_dt);
    if (out_dt == KB_DT_F32) { if (narrow) KB_COMBINE(float, bf16); else KB_COMBINE(float, float); }
    else if (out_dt == KB_DT_BF16) { if (narrow) KB_COMBINE(bf16, bf16); else KB_COMBINE(bf16, float); }
    else return fail("moe_combine: output dtype code %d is not known", out_dt);
#undef KB_COMBINE
    return check_launch("moe_combine");
}
