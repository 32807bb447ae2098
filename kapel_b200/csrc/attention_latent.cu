// Attention of all query heads over one cached line a position (a latent that is key and value at
// once): bfloat16 on tensor cores (mma.sync m16n8k16), for prompt portions and for single tokens.
//
// The cache has one kv head; a line holds d components, of which the first dv are the value. Every
// query head of a token reads the same lines, so a tile of 64 (token, head) rows shares each key it
// fetches: one block = up to 64 rows of one request (64 / heads tokens, or one token and a slice of
// 64 heads) x one chunk of keys (a launch's choice: the row-wise kernel's 256 for single tokens, where
// many blocks must share a long history; longer for prompts, which have tiles enough), with the slot
// numbers, partial sums and merge of the row-wise kernel (`combine_kernel`, which also adds the sink's term). Within a chunk the keys come 32 at a time into shared memory (16-byte asynchronous copies
// through the block table, the next 32 while these are multiplied); eight warps: four groups of 16 rows, and for each group two warps that each own half
// of the value's columns. Both compute the group's 16 x 32 scores (Q from shared memory as the A
// operand, the keys' lines as the B operand: a line is a column of K^T; both by ldmatrix), take the running maximum and
// the weights in 32-bit, and turn the weights into the A operand of the second product in registers;
// the lines, now as rows of V, come as its B operand by ldmatrix with a transpose. Scores, maxima,
// sums and the output accumulate in 32-bit. A key is seen by a row when it lies before the row's
// count (causal); a row that sees nothing in a chunk writes nothing for it.
#include "attention_rows.cuh"

namespace kb {

typedef __nv_bfloat16 bf16;

constexpr int LM_ROWS = 64;
constexpr int LM_KEYS = 32;
constexpr int LM_THREADS = 256;
constexpr int LM_MAX_NT = 32;          // tiles of 8 value columns a warp holds: dv <= 2 * 8 * 32

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

__global__ void __launch_bounds__(LM_THREADS, 1)
latent_mma_kernel(const AttParams p, const int* __restrict__ entry_start, const int* __restrict__ entry_end, int tokens_per_tile,
                  int heads_per_tile, int head_slices) {
    extern __shared__ __align__(16) unsigned char lm_smem[];
    const int d = p.d, dv = p.dv, H = p.hq;
    const int ld = d + 8;                                       // elements between rows in shared memory: 16-byte rows, banks spread
    bf16* sq = reinterpret_cast<bf16*>(lm_smem);                // [LM_ROWS][ld]
    bf16* sk = sq + (size_t)LM_ROWS * ld;                       // [2][LM_KEYS][ld]
    int* sline = reinterpret_cast<int*>(sk + (size_t)2 * LM_KEYS * ld);  // [2][LM_KEYS]
    int* scount = sline + 2 * LM_KEYS;                          // [LM_ROWS]: the count of each row's token, 0 for a row of no token

    const int entry = blockIdx.y, z = blockIdx.z;
    // the last tiles of a request see the most keys: they go first, so that the short ones fill the launch's end
    const int flipped = gridDim.x - 1 - blockIdx.x;
    const int tile = flipped / head_slices, hslice = flipped - tile * head_slices;
    const int e0 = entry_start[entry], e1 = entry_end[entry];
    const int r0 = e0 + tile * tokens_per_tile;
    if (r0 >= e1) return;
    const int ntok = min(tokens_per_tile, e1 - r0);
    const int h0 = hslice * heads_per_tile;
    const int nheads = min(heads_per_tile, H - h0);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gid = lane >> 2, t4 = lane & 3;
    const int group = warp & 3, half = warp >> 2;
    const int half_cols = dv >> 1;
    const int ntiles = half_cols >> 3;
    const int col0 = half * half_cols;

    // the rows' queries and counts
    const bf16* qg = static_cast<const bf16*>(p.q);
    const int nvec = d >> 3;
    for (int idx = tid; idx < LM_ROWS * nvec; idx += LM_THREADS) {
        const int rr = idx / nvec, v = idx - rr * nvec;
        const int t = rr / heads_per_tile, hh = rr - t * heads_per_tile;
        uint4 val = make_uint4(0u, 0u, 0u, 0u);
        if (t < ntok && hh < nheads) val = *reinterpret_cast<const uint4*>(qg + ((size_t)(r0 + t) * H + h0 + hh) * d + v * 8);
        *reinterpret_cast<uint4*>(sq + (size_t)rr * ld + v * 8) = val;
    }
    for (int rr = tid; rr < LM_ROWS; rr += LM_THREADS) {
        const int t = rr / heads_per_tile, hh = rr - t * heads_per_tile;
        scount[rr] = (t < ntok && hh < nheads) ? p.row_count[r0 + t] : 0;
    }
    __syncthreads();

    const int row_a = group * 16 + gid, row_b = row_a + 8;      // this thread's two rows of the tile
    const int count_a = scount[row_a], count_b = scount[row_b];
    const int most = p.row_count[r0 + ntok - 1];                // counts rise along a request's rows
    const int lo = z * p.chunk, hi = min(most, (z + 1) * p.chunk);

    float o[LM_MAX_NT][4];
#pragma unroll
    for (int j = 0; j < LM_MAX_NT; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;

    const bf16* kt = static_cast<const bf16*>(p.k_table);
    // The keys of a step come by asynchronous copies, the next step's while this one's are multiplied: two buffers.
    auto fetch = [&](int k0, int buf) {
        bf16* dst = sk + (size_t)buf * LM_KEYS * ld;
        for (int idx = tid; idx < LM_KEYS * nvec; idx += LM_THREADS) {
            const int key = idx / nvec, v = idx - key * nvec;
            const int pos = k0 + key;
            int line = -1;
            if (pos < hi) {
                const int lp = pos / p.page_size;
                const int page = lp < p.table_width ? p.block_table[(size_t)entry * p.table_width + lp] : -1;
                if (page >= 0 && page < p.n_pages) line = page * p.page_size + pos % p.page_size;
            }
            if (v == 0) sline[buf * LM_KEYS + key] = line;
            bf16* to = dst + (size_t)key * ld + v * 8;
            if (line >= 0) {
                const uint32_t to32 = (uint32_t)__cvta_generic_to_shared(to);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(to32), "l"(kt + kv_row(line, 0, 1, p.page_size) * d + v * 8) : "memory");
            } else {
                *reinterpret_cast<uint4*>(to) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (lo < hi) fetch(lo, 0);
    int turn = 0;
    for (int k0 = lo; k0 < hi; k0 += LM_KEYS, turn ^= 1) {
        if (k0 + LM_KEYS < hi) {
            fetch(k0 + LM_KEYS, turn ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const bf16* skb = sk + (size_t)turn * LM_KEYS * ld;
        const int* slineb = sline + turn * LM_KEYS;

        // ---- scores of 16 rows x 32 keys
        float s[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
        // operands by ldmatrix: Q's 16 x 16 piece as four 8 x 8 matrices in the A operand's order; the lines of two
        // 8-key tiles (keys are the matrices' rows, so no transpose) as b0, b1 of one tile and b0, b1 of the next
        const uint32_t qaddr = (uint32_t)__cvta_generic_to_shared(sq + (size_t)(group * 16 + (lane & 15)) * ld + (lane >> 4) * 8);
        const uint32_t kaddr = (uint32_t)__cvta_generic_to_shared(skb + (size_t)((lane >> 4) * 8 + (lane & 7)) * ld + ((lane >> 3) & 1) * 8);
        // two sets of sums taking the 16-component steps in turn: eight chains of products in flight instead of four
        float s2[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) s2[nt][0] = s2[nt][1] = s2[nt][2] = s2[nt][3] = 0.f;
        for (int kk = 0; kk < d; kk += 32) {
            uint32_t a[4], b[4], c[4];
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]) : "r"(qaddr + kk * 2));
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]) : "r"(kaddr + kk * 2));
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]) : "r"(kaddr + (16 * ld + kk) * 2));
            mma_bf16(s[0], a, b[0], b[1]);
            mma_bf16(s[1], a, b[2], b[3]);
            mma_bf16(s[2], a, c[0], c[1]);
            mma_bf16(s[3], a, c[2], c[3]);
            if (kk + 16 < d) {
                uint32_t a2[4], b2[4], c2[4];
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(a2[0]), "=r"(a2[1]), "=r"(a2[2]), "=r"(a2[3]) : "r"(qaddr + (kk + 16) * 2));
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(b2[0]), "=r"(b2[1]), "=r"(b2[2]), "=r"(b2[3]) : "r"(kaddr + (kk + 16) * 2));
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(c2[0]), "=r"(c2[1]), "=r"(c2[2]), "=r"(c2[3]) : "r"(kaddr + (16 * ld + kk + 16) * 2));
                mma_bf16(s2[0], a2, b2[0], b2[1]);
                mma_bf16(s2[1], a2, b2[2], b2[3]);
                mma_bf16(s2[2], a2, c2[0], c2[1]);
                mma_bf16(s2[3], a2, c2[2], c2[3]);
            }
        }
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int c = 0; c < 4; ++c) s[nt][c] += s2[nt][c];
        // ---- mask, running maximum, weights
        float top_a = m_a, top_b = m_b;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int key = k0 + nt * 8 + 2 * t4 + (c & 1);
                const bool seen = key < ((c & 2) ? count_b : count_a) && slineb[nt * 8 + 2 * t4 + (c & 1)] >= 0;
                s[nt][c] = seen ? s[nt][c] * p.scale : -INFINITY;
                if (c & 2) top_b = fmaxf(top_b, s[nt][c]);
                else top_a = fmaxf(top_a, s[nt][c]);
            }
        }
        top_a = fmaxf(top_a, __shfl_xor_sync(0xffffffffu, top_a, 1));
        top_a = fmaxf(top_a, __shfl_xor_sync(0xffffffffu, top_a, 2));
        top_b = fmaxf(top_b, __shfl_xor_sync(0xffffffffu, top_b, 1));
        top_b = fmaxf(top_b, __shfl_xor_sync(0xffffffffu, top_b, 2));
        const float fade_a = m_a == -INFINITY ? 1.f : __expf(m_a - top_a);     // a row that has seen nothing yet holds zeros
        const float fade_b = m_b == -INFINITY ? 1.f : __expf(m_b - top_b);
        m_a = top_a;
        m_b = top_b;
        float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float top = (c & 2) ? top_b : top_a;
                const float w = s[nt][c] == -INFINITY ? 0.f : __expf(s[nt][c] - top);
                s[nt][c] = w;
                if (c & 2) sum_b += w;
                else sum_a += w;
            }
        }
        l_a = l_a * fade_a + sum_a;                             // a thread's share of the row's sum; the four shares meet at the end
        l_b = l_b * fade_b + sum_b;
#pragma unroll
        for (int j = 0; j < LM_MAX_NT; ++j) {
            if (j < ntiles) {
                o[j][0] *= fade_a;
                o[j][1] *= fade_a;
                o[j][2] *= fade_b;
                o[j][3] *= fade_b;
            }
        }
        // ---- weights x values: the weights as the A operand, 16 keys a step
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
            uint32_t a[4];
            a[0] = pack_bf16(s[2 * ks][0], s[2 * ks][1]);
            a[1] = pack_bf16(s[2 * ks][2], s[2 * ks][3]);
            a[2] = pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]);
            a[3] = pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3]);
            const uint32_t row_addr = (uint32_t)__cvta_generic_to_shared(skb + (size_t)(ks * 16 + (lane & 15)) * ld + col0);
#pragma unroll
            for (int j = 0; j < LM_MAX_NT; ++j) {
                if (j < ntiles) {
                    uint32_t b0, b1;
                    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(row_addr + j * 16));
                    mma_bf16(o[j], a, b0, b1);
                }
            }
        }
        __syncthreads();                                        // this buffer is written again by the step after the next
    }

    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);

#pragma unroll
    for (int which = 0; which < 2; ++which) {
        const int rr = which ? row_b : row_a;
        const int t = rr / heads_per_tile, hh = rr - t * heads_per_tile;
        if (t >= ntok || hh >= nheads) continue;
        const int count = which ? count_b : count_a;
        const size_t r = (size_t)(r0 + t);
        const int h = h0 + hh;
        const float m = which ? m_b : m_a, l = which ? l_b : l_a;
        if (count <= 0) {                                       // a row that sees nothing at all: zeros, from the first chunk's block
            if (z == 0) {
                bf16* dst = static_cast<bf16*>(p.out) + (r * H + h) * dv + col0;
                for (int j = 0; j < ntiles; ++j) *reinterpret_cast<uint32_t*>(dst + j * 8 + 2 * t4) = 0u;
            }
            continue;
        }
        if (count <= lo) continue;                              // nothing of this chunk is before the row
        if (p.slots == 1) {
            float inv = l > 0.f ? 1.f / l : 0.f;
            if (p.sinks != nullptr) {                           // the weights were taken against the keys' maximum m
                const float sink = p.sinks[h];
                const float top = fmaxf(m, sink);
                const float wk = m == -INFINITY ? 0.f : __expf(m - top);
                inv = wk / (l * wk + __expf(sink - top));
            }
            bf16* dst = static_cast<bf16*>(p.out) + (r * H + h) * dv + col0;
#pragma unroll
            for (int j = 0; j < LM_MAX_NT; ++j)
                if (j < ntiles) *reinterpret_cast<uint32_t*>(dst + j * 8 + 2 * t4) = pack_bf16(o[j][2 * which] * inv, o[j][2 * which + 1] * inv);
        } else {
            float* dst = p.partial + ((r * H + h) * p.slots + z) * (dv + 2);
#pragma unroll
            for (int j = 0; j < LM_MAX_NT; ++j)
                if (j < ntiles) {
                    dst[col0 + j * 8 + 2 * t4] = o[j][2 * which];
                    dst[col0 + j * 8 + 2 * t4 + 1] = o[j][2 * which + 1];
                }
            if (half == 0 && t4 == 0) {
                dst[dv] = m;
                dst[dv + 1] = l;
            }
        }
    }
}

}  // namespace kb

using namespace kb;

// Whether the kernel takes these sizes: lines of whole 16-component steps, values that split into two
// halves of whole 8-column tiles a warp can hold.
extern "C" int kb_latent_attention_mma_takes(int d, int dv) {
    if (d <= 0 || dv <= 0 || dv > d || d % 16 || dv % 16 || dv > 2 * 8 * LM_MAX_NT) return 0;
    const size_t smem = ((size_t)LM_ROWS + 2 * LM_KEYS) * (d + 8) * sizeof(bf16) + (2 * LM_KEYS + LM_ROWS) * sizeof(int);
    return smem <= 200 * 1024 ? 1 : 0;
}

// q [rows, hq, d], table [pages, 1, page_size, d] (a line's first dv components are its value), out [rows, hq, dv]: bfloat16.
// entry_start / entry_end [entries]: the rows of each request; `longest`: the most rows any request brings.
// `chunk`: keys a slot holds, `slots` >= ceil(longest count / chunk).
// scratch: kb_paged_attention_scratch_floats(rows, hq, dv, slots) floats when slots > 1.
extern "C" int kb_latent_attention_mma(void* out, const void* q, const void* table, const int* block_table, const int* row_count,
                                       const int* entry_start, const int* entry_end, int entries, int longest, int rows, int hq,
                                       int d, int dv, int page_size, int table_width, int n_pages, int slots, int chunk, float scale,
                                       float* scratch, const float* sinks, void* stream) {
    KB_REQUIRE(chunk >= LM_KEYS && chunk % LM_KEYS == 0, "latent_attention_mma: chunks of %d keys (a multiple of %d)", chunk, LM_KEYS);
    KB_REQUIRE(rows >= 0 && entries >= 0 && hq > 0 && longest >= 0, "latent_attention_mma: rows %d, requests %d, heads %d, longest %d", rows, entries, hq, longest);
    KB_REQUIRE(kb_latent_attention_mma_takes(d, dv), "latent_attention_mma: lines of %d with values of %d are not taken (multiples of 16, values at most %d)", d, dv, 2 * 8 * LM_MAX_NT);
    KB_REQUIRE(page_size > 0 && table_width > 0 && n_pages > 0, "latent_attention_mma: page_size %d, table width %d, pages %d", page_size, table_width, n_pages);
    KB_REQUIRE(slots >= 1 && slots <= 65535 && (slots == 1 || scratch != nullptr), "latent_attention_mma: %d chunk slots (with scratch memory beyond one)", slots);
    KB_REQUIRE(out && q && table && block_table && row_count && entry_start && entry_end, "latent_attention_mma: a null input");
    KB_REQUIRE((((uintptr_t)q | (uintptr_t)table | (uintptr_t)out) & 15) == 0, "latent_attention_mma: tensors must be 16-byte aligned");
    if (rows == 0 || entries == 0 || longest == 0) return 0;
    AttParams p;
    p.q = q; p.k_table = table; p.v_table = table; p.block_table = block_table; p.row_entry = nullptr; p.row_count = row_count;
    p.out = out; p.partial = slots > 1 ? scratch : nullptr; p.rows = rows; p.hq = hq; p.hkv = 1; p.d = d; p.page_size = page_size;
    p.table_width = table_width; p.n_pages = n_pages; p.dv = dv; p.v_stride = d; p.sinks = sinks; p.vec = 1; p.window = 0; p.keep = 0;
    p.keep_slots = 0; p.block = 0; p.slots = slots; p.chunk = chunk; p.scale = scale; p.cap = 0.f;
    const int heads_per_tile = hq < LM_ROWS ? hq : LM_ROWS;
    const int head_slices = (hq + heads_per_tile - 1) / heads_per_tile;
    const int tokens_per_tile = LM_ROWS / heads_per_tile;
    const long long tiles = (long long)((longest + tokens_per_tile - 1) / tokens_per_tile) * head_slices;
    KB_REQUIRE(tiles <= 0x7fffffffll && entries <= 65535, "latent_attention_mma: too many tiles or requests for one launch");
    const size_t smem = ((size_t)LM_ROWS + 2 * LM_KEYS) * (d + 8) * sizeof(bf16) + (2 * LM_KEYS + LM_ROWS) * sizeof(int);
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(latent_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
            return fail("latent_attention_mma: cannot have 200 KB of shared memory");
        attr_set = true;
    }
    cudaStream_t s = (cudaStream_t)stream;
    latent_mma_kernel<<<dim3((unsigned)tiles, entries, slots), LM_THREADS, smem, s>>>(p, entry_start, entry_end, tokens_per_tile, heads_per_tile, head_slices);
    if (int e = check_launch("latent_attention_mma")) return e;
    if (slots > 1) {
        combine_kernel<bf16><<<dim3(rows, hq), 128, 0, s>>>(p);
        return check_launch("latent_attention_mma combine");
    }
    return 0;
}
