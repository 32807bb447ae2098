// Attention over a sliding window plus pooled blocks with mixed heads, for prompt portions, on
// tensor cores (mma.sync m16n8k16, bfloat16 operands, 32-bit scores, softmax, mix and sums).
//
// The mix (w'_h = sum_g talk[h, g] w_g) needs every head's normalised weight of a (query, key) pair, so
// a block takes up to 16 tokens of one request with ALL query heads and walks the keys twice, as two
// launches:
//   mode 1  scores of every head, 16 or 32 keys a step; each (token, head) keeps its running maximum
//           and sum, which go to a small table [rows, heads, 2];
//   mode 2  a block (tile, 8 output heads): the scores of every head again, normalised with the table's
//           maximum and sum; a thread holds all heads' weights of its (token, key) pairs in registers,
//           mixes them for the block's output heads and leaves them in shared memory as bfloat16;
//           each warp multiplies one output head's mixed weights with its kv head's values.
// Where scratch memory allows, the scores are kept between the launches instead: `pooled_stats_kernel` (a
// block a tile and 8 heads: only their queries and their kv heads' keys) leaves the statistics and the masked
// scores, and `pooled_mix_kernel` (a block a tile and 8 or 16 output heads) fetches a step's scores of all
// heads by cp.async, with the values of its heads' kv heads, and normalises, mixes and multiplies: no
// queries, no keys, no score computed twice. `pooled_mma_kernel`'s two modes are what runs otherwise.
// Keys and values of a step lie in shared memory for all kv heads (the pooled means, 32-bit in their
// table, are rounded to bfloat16 on the way in); fragments come by ldmatrix. Which keys a token sees:
// the blocks b < floor((c - window) / pool) and the tokens [max(0, c - window), c), c the positions it
// has seen. Sizes: head sizes that are multiples of 16, values up to 128 wide, up to 32 query heads.
#include "common.cuh"

namespace kb {

typedef __nv_bfloat16 bf16;

constexpr int PM_THREADS = 512;
constexpr int PM_WARPS = PM_THREADS / 32;
constexpr int PM_ROWS = 16;           // tokens a tile
constexpr int PM_HEADS = 8;           // output heads a block in mode 2: one a warp
constexpr int PM_PAD = 8;             // elements of padding a shared-memory row (16 bytes)

struct PooledMmaParams {
    const bf16* q;             // [rows, hq, d]
    const bf16* k_table;       // [pages, hkv, page_size, d]
    const bf16* v_table;       // [pages, hkv, page_size, dv]
    const float* pooled;       // [slots, max_blocks, hkv, d + dv]
    const int* block_table;    // [entries, table_width]
    const int* row_count;      // [rows]
    const int* tile_entry;     // [tiles]
    const int* tile_row0;      // [tiles]
    const int* tile_nq;        // [tiles] tokens of the tile (<= 16)
    const int* slots;          // [entries]
    const float* talk;         // [hq, hq] or null
    const float* temp;         // [hq] or null
    bf16* out;                 // [rows, hq, dv]
    float* stats;              // [rows, hq, 2]
    float* kept;               // [tiles, kept_steps, hq, 16, 16] the first launch's scores in runs of 16 keys (-inf: not seen), or null
    int kept_steps;            // runs of 16 keys a tile has room for (an even number)
    long long slot_stride;
    int hq, hkv, d, dv, page_size, table_width, n_pages, n_slots, max_blocks;
    int window, pool;
    int ncv;                   // the most kv heads any block's output heads read values of
    int ncv_mix;               // the same for the blocks of the launch that reads kept scores (8 or 16 heads a block)
    int mode;
    float scale;
};

struct PmLayout { unsigned q, k, v, pp, ss, m, il, talk, temp, ints, total; };

__host__ __device__ inline unsigned pm_take(unsigned& at, size_t bytes) {
    const unsigned o = at;
    at += (unsigned)((bytes + 15) & ~(size_t)15);
    return o;
}

__host__ __device__ inline PmLayout pm_layout(int hq, int hkv, int d, int dv, int ncv, int nk, int stages) {
    PmLayout L;
    unsigned at = 0;
    L.q = pm_take(at, (size_t)PM_ROWS * (hq * d + PM_PAD) * 2);
    L.k = pm_take(at, (size_t)stages * hkv * nk * (d + PM_PAD) * 2);
    L.v = pm_take(at, (size_t)stages * ncv * nk * (dv + PM_PAD) * 2);
    L.pp = pm_take(at, (size_t)PM_HEADS * PM_ROWS * (nk + PM_PAD) * 2);
    L.ss = pm_take(at, (size_t)hq * PM_ROWS * (nk + 1) * 4);
    L.m = pm_take(at, (size_t)hq * PM_ROWS * 4);
    L.il = pm_take(at, (size_t)hq * PM_ROWS * 4);
    L.talk = pm_take(at, (size_t)PM_HEADS * 32 * 4);
    L.temp = pm_take(at, (size_t)hq * 4);
    L.ints = pm_take(at, (size_t)3 * PM_ROWS * 4);
    L.total = at;
    return L;
}

__device__ __forceinline__ void pm_ldmatrix_x4(uint32_t (&r)[4], const bf16* p) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void pm_ldmatrix_x4_trans(uint32_t (&r)[4], const bf16* p) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void pm_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void pm_cp_async16(void* smem, const void* gmem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void pm_cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void pm_cp_async_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }
__device__ __forceinline__ uint32_t pm_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// NK: keys a step; HMAX: the most query heads (weights a thread holds); DVMAX: the widest values;
// STAGES: 2 when shared memory holds two steps' keys and values (the next step's arrive while this one is computed).
template <int NK, int HMAX, int DVMAX, int STAGES>
__global__ void __launch_bounds__(PM_THREADS, 1)
pooled_mma_kernel(const PooledMmaParams p) {
    extern __shared__ __align__(16) unsigned char pm_smem[];
    const int hq = p.hq, hkv = p.hkv, d = p.d, dv = p.dv, group = p.hq / p.hkv;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int t = gridDim.x - 1 - blockIdx.x;                // later tiles see more keys: they start first
    const int entry = p.tile_entry[t], r0 = p.tile_row0[t], nq = min(p.tile_nq[t], PM_ROWS);
    const int h0 = p.mode == 2 ? blockIdx.y * PM_HEADS : 0;
    const int nh = p.mode == 2 ? min(PM_HEADS, hq - h0) : 0;
    const int c_lo = h0 / group;
    const int ncv = p.mode == 2 ? (h0 + nh - 1) / group - c_lo + 1 : 0;
    const PmLayout L = pm_layout(hq, hkv, d, dv, p.ncv, NK, STAGES);
    bf16* sQ = reinterpret_cast<bf16*>(pm_smem + L.q);
    bf16* sK = reinterpret_cast<bf16*>(pm_smem + L.k);
    bf16* sV = reinterpret_cast<bf16*>(pm_smem + L.v);
    bf16* pp = reinterpret_cast<bf16*>(pm_smem + L.pp);
    float* ss = reinterpret_cast<float*>(pm_smem + L.ss);
    float* s_m = reinterpret_cast<float*>(pm_smem + L.m);
    float* s_il = reinterpret_cast<float*>(pm_smem + L.il);     // mode 1: the running sum; mode 2: 1 / sum
    float* s_talk = reinterpret_cast<float*>(pm_smem + L.talk);
    float* s_temp = reinterpret_cast<float*>(pm_smem + L.temp);
    int* s_cnt = reinterpret_cast<int*>(pm_smem + L.ints);
    int* s_first = s_cnt + PM_ROWS;
    int* s_nb = s_first + PM_ROWS;
    const int ldq = hq * d + PM_PAD, ldk = d + PM_PAD, ldv = dv + PM_PAD, ldp = NK + PM_PAD, lds = NK + 1;
    const int wide = d + dv;
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);

    if (tid < PM_ROWS) {
        int c = tid < nq ? p.row_count[r0 + tid] : 0;
        c = max(c, 0);
        const bool past = p.window > 0 && c > p.window;
        s_cnt[tid] = c;
        s_first[tid] = past ? c - p.window : 0;
        s_nb[tid] = (past && p.pool > 0) ? min((c - p.window) / p.pool, p.max_blocks) : 0;
    }
    {
        const int qch = hq * d / 8;
        for (int idx = tid; idx < PM_ROWS * qch; idx += PM_THREADS) {
            const int i = idx / qch, ch = idx - i * qch;
            const uint4 v = i < nq ? *reinterpret_cast<const uint4*>(p.q + (size_t)(r0 + i) * hq * d + ch * 8) : zero4;
            *reinterpret_cast<uint4*>(sQ + (size_t)i * ldq + ch * 8) = v;
        }
    }
    for (int i = tid; i < hq; i += PM_THREADS) s_temp[i] = (p.temp != nullptr ? p.temp[i] : 1.f) * p.scale;
    for (int i = tid; i < nh * HMAX; i += PM_THREADS) {     // rows as wide as a thread's weights, zeros past the last head
        const int h = h0 + i / HMAX, g = i % HMAX;
        s_talk[i] = g >= hq ? 0.f : (p.talk != nullptr ? p.talk[(size_t)h * hq + g] : (h == g ? 1.f : 0.f));
    }
    for (int i = tid; i < hq * PM_ROWS; i += PM_THREADS) {
        const int g = i / PM_ROWS, r = i - g * PM_ROWS;
        if (p.mode == 1) {
            s_m[i] = -INFINITY;
            s_il[i] = 0.f;
        } else if (r < nq) {
            const float* st = p.stats + ((size_t)(r0 + r) * hq + g) * 2;
            const float l = st[1];
            s_m[i] = st[0];
            s_il[i] = l > 0.f ? 1.f / l : 0.f;
        } else {
            s_m[i] = 0.f;
            s_il[i] = 0.f;
        }
    }
    __syncthreads();
    int nb_max = 0, first_min = 0x7fffffff, c_max = 0;
    for (int i = 0; i < nq; ++i) {
        nb_max = max(nb_max, s_nb[i]);
        first_min = min(first_min, s_first[i]);
        c_max = max(c_max, s_cnt[i]);
    }
    const int n_keys = c_max > 0 ? nb_max + (c_max - first_min) : 0;
    const int slot = p.slots[entry];
    const float* pooled = p.pooled + (size_t)((slot > 0 && slot < p.n_slots) ? slot : 0) * p.slot_stride;
    const int* pages = p.block_table + (size_t)entry * p.table_width;

    // A thread's two rows of every score tile, as ranges of the key index: blocks [0, nb) and tokens [lo, hi).
    const int ia = lane >> 2, ib = ia + 8;
    const int nb_a = s_nb[ia], lo_a = nb_max + s_first[ia] - first_min, hi_a = nb_max + s_cnt[ia] - first_min;
    const int nb_b = s_nb[ib], lo_b = nb_max + s_first[ib] - first_min, hi_b = nb_max + s_cnt[ib] - first_min;
    // What every token of the tile sees (tokens come in the order of their positions).
    const int all_nb = s_nb[0], all_lo = nb_max + s_first[nq - 1] - first_min, all_hi = nb_max + s_cnt[0] - first_min;

    constexpr int OT = (DVMAX / 16 + 1) / 2;             // 16-wide value tiles a warp: two warps share an output head
    float o[2 * OT][4];
#pragma unroll
    for (int n = 0; n < 2 * OT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

    // A step's keys (all kv heads) and values (the kv heads of this block's output heads) into buffer `buf`:
    // PM_THREADS / NK threads a key look its page up once; token lines come by cp.async, the 32-bit block
    // means are rounded on the way, keys past the last are zeros.
    constexpr int TPK = PM_THREADS / NK;
    auto issue = [&](int j0, int buf) {
        const int jj = tid / TPK, sub = tid - jj * TPK;
        const int j = j0 + jj;
        bf16* kd = sK + (size_t)buf * hkv * NK * ldk + (size_t)jj * ldk;
        bf16* vd = sV + (size_t)buf * p.ncv * NK * ldv + (size_t)jj * ldv;
        long long row = -1;                                  // the token's row of kv head 0 in the tables
        if (j >= nb_max && j < n_keys) {
            const int pos = first_min + (j - nb_max);
            const int lp = pos / p.page_size;
            const int page = lp < p.table_width ? pages[lp] : -1;
            if (page >= 0 && page < p.n_pages) row = (long long)page * hkv * p.page_size + (pos - lp * p.page_size);
        }
        if (row >= 0) {
            for (int c = 0; c < hkv; ++c) {
                const bf16* src = p.k_table + (size_t)(row + (long long)c * p.page_size) * d;
                for (int ch = sub; ch * 8 < d; ch += TPK) pm_cp_async16(kd + (size_t)c * NK * ldk + ch * 8, src + ch * 8);
            }
            for (int cl = 0; cl < ncv; ++cl) {
                const bf16* src = p.v_table + (size_t)(row + (long long)(c_lo + cl) * p.page_size) * dv;
                for (int ch = sub; ch * 8 < dv; ch += TPK) pm_cp_async16(vd + (size_t)cl * NK * ldv + ch * 8, src + ch * 8);
            }
        } else if (j < nb_max) {
            for (int c = 0; c < hkv; ++c) {
                const float* src = pooled + ((size_t)j * hkv + c) * wide;
                for (int ch = sub; ch * 8 < d; ch += TPK) {
                    const float4 a = *reinterpret_cast<const float4*>(src + ch * 8), b = *reinterpret_cast<const float4*>(src + ch * 8 + 4);
                    *reinterpret_cast<uint4*>(kd + (size_t)c * NK * ldk + ch * 8) = make_uint4(pm_pack(a.x, a.y), pm_pack(a.z, a.w), pm_pack(b.x, b.y), pm_pack(b.z, b.w));
                }
            }
            for (int cl = 0; cl < ncv; ++cl) {
                const float* src = pooled + ((size_t)j * hkv + c_lo + cl) * wide + d;
                for (int ch = sub; ch * 8 < dv; ch += TPK) {
                    const float4 a = *reinterpret_cast<const float4*>(src + ch * 8), b = *reinterpret_cast<const float4*>(src + ch * 8 + 4);
                    *reinterpret_cast<uint4*>(vd + (size_t)cl * NK * ldv + ch * 8) = make_uint4(pm_pack(a.x, a.y), pm_pack(a.z, a.w), pm_pack(b.x, b.y), pm_pack(b.z, b.w));
                }
            }
        } else {
            for (int c = 0; c < hkv; ++c)
                for (int ch = sub; ch * 8 < d; ch += TPK) *reinterpret_cast<uint4*>(kd + (size_t)c * NK * ldk + ch * 8) = zero4;
            for (int cl = 0; cl < ncv; ++cl)
                for (int ch = sub; ch * 8 < dv; ch += TPK) *reinterpret_cast<uint4*>(vd + (size_t)cl * NK * ldv + ch * 8) = zero4;
        }
        pm_cp_async_commit();
    };

    if (STAGES == 2 && n_keys > 0) issue(0, 0);
    for (int j0 = 0; j0 < n_keys; j0 += NK) {
        const int buf = STAGES == 2 ? (j0 / NK) & 1 : 0;
        if (STAGES == 1) issue(j0, 0);
        pm_cp_async_wait_all();
        __syncthreads();                                     // the step's keys and values are in; everyone has left the step before
        if (STAGES == 2 && j0 + NK < n_keys) issue(j0 + NK, buf ^ 1);
        const bf16* bK = sK + (size_t)buf * hkv * NK * ldk;
        const bf16* bV = sV + (size_t)buf * p.ncv * NK * ldv;
        // ---- scores: an item is a head and 16 keys
        constexpr int NSUB = NK / 16;
        for (int item = warp; item < hq * NSUB; item += PM_WARPS) {
            const int g = item / NSUB, sub = item - g * NSUB;
            const int c = g / group;
            float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            const bf16* qa = sQ + (size_t)(lane & 15) * ldq + g * d + (lane >> 4) * 8;
            const bf16* kf = bK + ((size_t)c * NK + sub * 16 + (lane & 7) + ((lane >> 4) << 3)) * ldk + ((lane >> 3) & 1) * 8;
            for (int ks = 0; ks < d; ks += 16) {
                uint32_t a[4], b[4];
                pm_ldmatrix_x4(a, qa + ks);
                pm_ldmatrix_x4(b, kf + ks);
                pm_mma(acc[0], a, b[0], b[1]);
                pm_mma(acc[1], a, b[2], b[3]);
            }
            const float tg = s_temp[g];
            const int js = j0 + sub * 16;
            const bool whole = js + 16 <= all_nb || (js >= all_lo && js + 16 <= all_hi);     // every token sees all 16 keys
            float ma = 0.f, mb = 0.f, la = 1.f, lb = 1.f;
            if (p.mode == 2) {
                ma = s_m[g * PM_ROWS + ia]; la = s_il[g * PM_ROWS + ia];
                mb = s_m[g * PM_ROWS + ib]; lb = s_il[g * PM_ROWS + ib];
            }
            float* sa = ss + (size_t)(g * PM_ROWS + ia) * lds + sub * 16 + (lane & 3) * 2;
            float* sb = ss + (size_t)(g * PM_ROWS + ib) * lds + sub * 16 + (lane & 3) * 2;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int j = js + nt * 8 + (lane & 3) * 2 + e;
                    const bool seen_a = whole || j < nb_a || (j >= lo_a && j < hi_a);
                    const bool seen_b = whole || j < nb_b || (j >= lo_b && j < hi_b);
                    float va = acc[nt][e] * tg, vb = acc[nt][2 + e] * tg;
                    if (p.mode == 2) {                       // the normalised weight, from the first launch's maximum and sum
                        va = seen_a ? __expf(va - ma) * la : 0.f;
                        vb = seen_b ? __expf(vb - mb) * lb : 0.f;
                    } else {
                        va = seen_a ? va : -INFINITY;
                        vb = seen_b ? vb : -INFINITY;
                    }
                    sa[nt * 8 + e] = va;
                    sb[nt * 8 + e] = vb;
                }
        }
        __syncthreads();
        if (p.mode == 1) {
            // ---- every (head, token): the running maximum and sum
            for (int pr = tid; pr < hq * PM_ROWS; pr += PM_THREADS) {
                const float* row = ss + (size_t)pr * lds;
                float mx = -INFINITY;
#pragma unroll
                for (int jj = 0; jj < NK; ++jj) mx = fmaxf(mx, row[jj]);
                const float old = s_m[pr];
                const float top = fmaxf(old, mx);
                if (top != -INFINITY) {
                    float l = 0.f;
#pragma unroll
                    for (int jj = 0; jj < NK; ++jj) l += __expf(row[jj] - top);
                    s_il[pr] = (old == -INFINITY ? 0.f : s_il[pr] * __expf(old - top)) + l;
                    s_m[pr] = top;
                }
            }
            continue;                                        // the next step's first barrier stands between these reads and its scores
        }
        // ---- a thread takes (token, key) pairs: all heads' weights, mixed for this block's heads
        for (int e = tid; e < PM_ROWS * NK; e += PM_THREADS) {
            const int i = e / NK, jj = e - i * NK;
            float pg[HMAX];
#pragma unroll
            for (int g = 0; g < HMAX; ++g) pg[g] = g < hq ? ss[(size_t)(g * PM_ROWS + i) * lds + jj] : 0.f;
            for (int hl = 0; hl < nh; ++hl) {
                const float4* tr = reinterpret_cast<const float4*>(s_talk + hl * HMAX);
                float w = 0.f;
#pragma unroll
                for (int g4 = 0; g4 < HMAX / 4; ++g4) {
                    const float4 t4 = tr[g4];
                    w = fmaf(t4.x, pg[4 * g4], w); w = fmaf(t4.y, pg[4 * g4 + 1], w);
                    w = fmaf(t4.z, pg[4 * g4 + 2], w); w = fmaf(t4.w, pg[4 * g4 + 3], w);
                }
                pp[(size_t)(hl * PM_ROWS + i) * ldp + jj] = __float2bfloat16(w);
            }
        }
        __syncthreads();
        // ---- two warps an output head: its mixed weights times halves of its kv head's values
        if (warp < 2 * nh) {
            const int hl = warp >> 1, half = warp & 1;
            const int cl = (h0 + hl) / group - c_lo;
            const bf16* pa = pp + (size_t)(hl * PM_ROWS + (lane & 15)) * ldp + (lane >> 4) * 8;
            const bf16* vf = bV + ((size_t)cl * NK + (lane & 7) + ((lane >> 3) & 1) * 8) * ldv + (lane >> 4) * 8 + half * OT * 16;
#pragma unroll
            for (int kk = 0; kk < NK; kk += 16) {
                uint32_t a[4];
                pm_ldmatrix_x4(a, pa + kk);
#pragma unroll
                for (int n2 = 0; n2 < OT; ++n2) {
                    if ((half * OT + n2) * 16 < dv) {
                        uint32_t b[4];
                        pm_ldmatrix_x4_trans(b, vf + (size_t)kk * ldv + n2 * 16);
                        pm_mma(o[2 * n2], a, b[0], b[1]);
                        pm_mma(o[2 * n2 + 1], a, b[2], b[3]);
                    }
                }
            }
        }
        if (STAGES == 1) __syncthreads();                    // before the next step's keys and values overwrite these
    }

    if (p.mode == 1) {
        for (int pr = tid; pr < hq * PM_ROWS; pr += PM_THREADS) {
            const int g = pr / PM_ROWS, i = pr - g * PM_ROWS;
            if (i < nq) {
                float* st = p.stats + ((size_t)(r0 + i) * hq + g) * 2;
                st[0] = s_m[pr];
                st[1] = s_il[pr];
            }
        }
        return;
    }
    if (warp < 2 * nh) {
        const int h = h0 + (warp >> 1), half = warp & 1;
#pragma unroll
        for (int n = 0; n < 2 * OT; ++n) {
            const int col = (half * OT * 2 + n) * 8 + (lane & 3) * 2;
            if (col < dv) {
                const int i = lane >> 2;
                if (i < nq) *reinterpret_cast<uint32_t*>(p.out + ((size_t)(r0 + i) * hq + h) * dv + col) = pm_pack(o[n][0], o[n][1]);
                if (i + 8 < nq) *reinterpret_cast<uint32_t*>(p.out + ((size_t)(r0 + i + 8) * hq + h) * dv + col) = pm_pack(o[n][2], o[n][3]);
            }
        }
    }
}

// The first launch when scores are kept: a block (tile, 8 heads) computes its heads' scores only (their queries, their
// kv heads' keys), keeps each (token, head)'s running maximum and sum for the table, and writes the masked scores to
// scratch memory in runs of 16 keys [tile, run, head, token, 16]. Heads are independent here: no block repeats another's work.
struct PmStatsLayout { unsigned q, k, ss, m, l, temp, ints, total; };

__host__ __device__ inline PmStatsLayout pm_stats_layout(int hq, int d, int ncv, int nk, int stages) {
    PmStatsLayout L;
    unsigned at = 0;
    const int heads = hq < PM_HEADS ? hq : PM_HEADS;
    L.q = pm_take(at, (size_t)PM_ROWS * (heads * d + PM_PAD) * 2);
    L.k = pm_take(at, (size_t)stages * ncv * nk * (d + PM_PAD) * 2);
    L.ss = pm_take(at, (size_t)heads * PM_ROWS * (nk + 1) * 4);
    L.m = pm_take(at, (size_t)heads * PM_ROWS * 4);
    L.l = pm_take(at, (size_t)heads * PM_ROWS * 4);
    L.temp = pm_take(at, (size_t)heads * 4);
    L.ints = pm_take(at, (size_t)3 * PM_ROWS * 4);
    L.total = at;
    return L;
}

template <int NK, int STAGES>
__global__ void __launch_bounds__(PM_THREADS, 1)
pooled_stats_kernel(const PooledMmaParams p) {
    extern __shared__ __align__(16) unsigned char pm_smem[];
    const int hq = p.hq, hkv = p.hkv, d = p.d, dv = p.dv, group = p.hq / p.hkv;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int t = gridDim.x - 1 - blockIdx.x;
    const int entry = p.tile_entry[t], r0 = p.tile_row0[t], nq = min(p.tile_nq[t], PM_ROWS);
    const int h0 = blockIdx.y * PM_HEADS;
    const int nh = min(PM_HEADS, hq - h0);
    const int c_lo = h0 / group;
    const int ncv = (h0 + nh - 1) / group - c_lo + 1;
    const PmStatsLayout L = pm_stats_layout(hq, d, p.ncv, NK, STAGES);
    bf16* sQ = reinterpret_cast<bf16*>(pm_smem + L.q);
    bf16* sK = reinterpret_cast<bf16*>(pm_smem + L.k);
    float* ss = reinterpret_cast<float*>(pm_smem + L.ss);
    float* s_m = reinterpret_cast<float*>(pm_smem + L.m);
    float* s_l = reinterpret_cast<float*>(pm_smem + L.l);
    float* s_temp = reinterpret_cast<float*>(pm_smem + L.temp);
    int* s_cnt = reinterpret_cast<int*>(pm_smem + L.ints);
    int* s_first = s_cnt + PM_ROWS;
    int* s_nb = s_first + PM_ROWS;
    const int ldq = min(hq, PM_HEADS) * d + PM_PAD, ldk = d + PM_PAD, lds = NK + 1;
    const int wide = d + dv;
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);

    if (tid < PM_ROWS) {
        int c = tid < nq ? p.row_count[r0 + tid] : 0;
        c = max(c, 0);
        const bool past = p.window > 0 && c > p.window;
        s_cnt[tid] = c;
        s_first[tid] = past ? c - p.window : 0;
        s_nb[tid] = (past && p.pool > 0) ? min((c - p.window) / p.pool, p.max_blocks) : 0;
    }
    {
        const int qch = nh * d / 8;
        for (int idx = tid; idx < PM_ROWS * qch; idx += PM_THREADS) {
            const int i = idx / qch, ch = idx - i * qch;
            const uint4 v = i < nq ? *reinterpret_cast<const uint4*>(p.q + ((size_t)(r0 + i) * hq + h0) * d + ch * 8) : zero4;
            *reinterpret_cast<uint4*>(sQ + (size_t)i * ldq + ch * 8) = v;
        }
    }
    for (int i = tid; i < nh; i += PM_THREADS) s_temp[i] = (p.temp != nullptr ? p.temp[h0 + i] : 1.f) * p.scale;
    for (int i = tid; i < nh * PM_ROWS; i += PM_THREADS) {
        s_m[i] = -INFINITY;
        s_l[i] = 0.f;
    }
    __syncthreads();
    int nb_max = 0, first_min = 0x7fffffff, c_max = 0;
    for (int i = 0; i < nq; ++i) {
        nb_max = max(nb_max, s_nb[i]);
        first_min = min(first_min, s_first[i]);
        c_max = max(c_max, s_cnt[i]);
    }
    const int n_keys = c_max > 0 ? nb_max + (c_max - first_min) : 0;
    const int slot = p.slots[entry];
    const float* pooled = p.pooled + (size_t)((slot > 0 && slot < p.n_slots) ? slot : 0) * p.slot_stride;
    const int* pages = p.block_table + (size_t)entry * p.table_width;
    const int ia = lane >> 2, ib = ia + 8;
    const int nb_a = s_nb[ia], lo_a = nb_max + s_first[ia] - first_min, hi_a = nb_max + s_cnt[ia] - first_min;
    const int nb_b = s_nb[ib], lo_b = nb_max + s_first[ib] - first_min, hi_b = nb_max + s_cnt[ib] - first_min;
    const int all_nb = s_nb[0], all_lo = nb_max + s_first[nq - 1] - first_min, all_hi = nb_max + s_cnt[0] - first_min;

    constexpr int TPK = PM_THREADS / NK;
    auto issue = [&](int j0, int buf) {
        const int jj = tid / TPK, sub = tid - jj * TPK;
        const int j = j0 + jj;
        bf16* kd = sK + (size_t)buf * p.ncv * NK * ldk + (size_t)jj * ldk;
        long long row = -1;
        if (j >= nb_max && j < n_keys) {
            const int pos = first_min + (j - nb_max);
            const int lp = pos / p.page_size;
            const int page = lp < p.table_width ? pages[lp] : -1;
            if (page >= 0 && page < p.n_pages) row = (long long)page * hkv * p.page_size + (pos - lp * p.page_size);
        }
        if (row >= 0) {
            for (int cl = 0; cl < ncv; ++cl) {
                const bf16* src = p.k_table + (size_t)(row + (long long)(c_lo + cl) * p.page_size) * d;
                for (int ch = sub; ch * 8 < d; ch += TPK) pm_cp_async16(kd + (size_t)cl * NK * ldk + ch * 8, src + ch * 8);
            }
        } else if (j < nb_max) {
            for (int cl = 0; cl < ncv; ++cl) {
                const float* src = pooled + ((size_t)j * hkv + c_lo + cl) * wide;
                for (int ch = sub; ch * 8 < d; ch += TPK) {
                    const float4 a = *reinterpret_cast<const float4*>(src + ch * 8), b = *reinterpret_cast<const float4*>(src + ch * 8 + 4);
                    *reinterpret_cast<uint4*>(kd + (size_t)cl * NK * ldk + ch * 8) = make_uint4(pm_pack(a.x, a.y), pm_pack(a.z, a.w), pm_pack(b.x, b.y), pm_pack(b.z, b.w));
                }
            }
        } else {
            for (int cl = 0; cl < ncv; ++cl)
                for (int ch = sub; ch * 8 < d; ch += TPK) *reinterpret_cast<uint4*>(kd + (size_t)cl * NK * ldk + ch * 8) = zero4;
        }
        pm_cp_async_commit();
    };

    if (STAGES == 2 && n_keys > 0) issue(0, 0);
    for (int j0 = 0; j0 < n_keys; j0 += NK) {
        const int buf = STAGES == 2 ? (j0 / NK) & 1 : 0;
        if (STAGES == 1) issue(j0, 0);
        pm_cp_async_wait_all();
        __syncthreads();                                     // the step's keys are in; everyone has left the step before
        if (STAGES == 2 && j0 + NK < n_keys) issue(j0 + NK, buf ^ 1);
        const bf16* bK = sK + (size_t)buf * p.ncv * NK * ldk;
        constexpr int NSUB = NK / 16;
        for (int item = warp; item < nh * NSUB; item += PM_WARPS) {
            const int gl = item / NSUB, sub = item - gl * NSUB;
            const int g = h0 + gl;
            const int cl = g / group - c_lo;
            float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            const bf16* qa = sQ + (size_t)(lane & 15) * ldq + gl * d + (lane >> 4) * 8;
            const bf16* kf = bK + ((size_t)cl * NK + sub * 16 + (lane & 7) + ((lane >> 4) << 3)) * ldk + ((lane >> 3) & 1) * 8;
            for (int ks = 0; ks < d; ks += 16) {
                uint32_t a[4], b[4];
                pm_ldmatrix_x4(a, qa + ks);
                pm_ldmatrix_x4(b, kf + ks);
                pm_mma(acc[0], a, b[0], b[1]);
                pm_mma(acc[1], a, b[2], b[3]);
            }
            const float tg = s_temp[gl];
            const int js = j0 + sub * 16;
            const bool whole = js + 16 <= all_nb || (js >= all_lo && js + 16 <= all_hi);
            float* sa = ss + (size_t)(gl * PM_ROWS + ia) * lds + sub * 16 + (lane & 3) * 2;
            float* sb = ss + (size_t)(gl * PM_ROWS + ib) * lds + sub * 16 + (lane & 3) * 2;
            float* run = p.kept + ((size_t)t * p.kept_steps + js / 16) * hq * PM_ROWS * 16;
            float* ka = run + (size_t)(g * PM_ROWS + ia) * 16 + (lane & 3) * 2;
            float* kb2 = run + (size_t)(g * PM_ROWS + ib) * 16 + (lane & 3) * 2;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                float va[2], vb[2];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int j = js + nt * 8 + (lane & 3) * 2 + e;
                    const bool seen_a = whole || j < nb_a || (j >= lo_a && j < hi_a);
                    const bool seen_b = whole || j < nb_b || (j >= lo_b && j < hi_b);
                    va[e] = seen_a ? acc[nt][e] * tg : -INFINITY;
                    vb[e] = seen_b ? acc[nt][2 + e] * tg : -INFINITY;
                    sa[nt * 8 + e] = va[e];
                    sb[nt * 8 + e] = vb[e];
                }
                *reinterpret_cast<float2*>(ka + nt * 8) = make_float2(va[0], va[1]);
                *reinterpret_cast<float2*>(kb2 + nt * 8) = make_float2(vb[0], vb[1]);
            }
        }
        __syncthreads();
        for (int pr = tid; pr < nh * PM_ROWS; pr += PM_THREADS) {
            const float* row = ss + (size_t)pr * lds;
            float mx = -INFINITY;
#pragma unroll
            for (int jj = 0; jj < NK; ++jj) mx = fmaxf(mx, row[jj]);
            const float old = s_m[pr];
            const float top = fmaxf(old, mx);
            if (top != -INFINITY) {
                float l = 0.f;
#pragma unroll
                for (int jj = 0; jj < NK; ++jj) l += __expf(row[jj] - top);
                s_l[pr] = (old == -INFINITY ? 0.f : s_l[pr] * __expf(old - top)) + l;
                s_m[pr] = top;
            }
        }
        // (the next step's first barrier stands between these reads and its scores)
    }
    for (int pr = tid; pr < nh * PM_ROWS; pr += PM_THREADS) {
        const int gl = pr / PM_ROWS, i = pr - gl * PM_ROWS;
        if (i < nq) {
            float* st = p.stats + ((size_t)(r0 + i) * hq + h0 + gl) * 2;
            st[0] = s_m[pr];
            st[1] = s_l[pr];
        }
    }
}

// The second launch when the first kept its scores: a block (tile, 8 output heads) fetches a step's scores of all
// heads (cp.async straight into shared memory, two buffers) and the values of its heads' kv heads, normalises,
// mixes and multiplies as above. No queries, no keys, no score is computed twice.
struct PmMixLayout { unsigned sc, v, pp, m, il, talk, ints, total; };

__host__ __device__ inline PmMixLayout pm_mix_layout(int hq, int dv, int ncv, int nk, int hb) {
    PmMixLayout L;
    unsigned at = 0;
    L.sc = pm_take(at, (size_t)2 * hq * PM_ROWS * (nk + 4) * 4);
    L.v = pm_take(at, (size_t)2 * ncv * nk * (dv + PM_PAD) * 2);
    L.pp = pm_take(at, (size_t)hb * PM_ROWS * (nk + PM_PAD) * 2);
    L.m = pm_take(at, (size_t)hq * PM_ROWS * 4);
    L.il = pm_take(at, (size_t)hq * PM_ROWS * 4);
    L.talk = pm_take(at, (size_t)hb * 32 * 4);
    L.ints = pm_take(at, (size_t)3 * PM_ROWS * 4);
    L.total = at;
    return L;
}

// HB: output heads a block, 8 (two warps a head, halves of the values) or 16 (a warp a head).
template <int NK, int HMAX, int DVMAX, int HB>
__global__ void __launch_bounds__(PM_THREADS, 1)
pooled_mix_kernel(const PooledMmaParams p) {
    extern __shared__ __align__(16) unsigned char pm_smem[];
    const int hq = p.hq, hkv = p.hkv, d = p.d, dv = p.dv, group = p.hq / p.hkv;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int t = gridDim.x - 1 - blockIdx.x;
    const int entry = p.tile_entry[t], r0 = p.tile_row0[t], nq = min(p.tile_nq[t], PM_ROWS);
    constexpr int SPLIT = PM_WARPS / HB;                  // warps an output head
    const int h0 = blockIdx.y * HB;
    const int nh = min(HB, hq - h0);
    const int c_lo = h0 / group;
    const int ncv = (h0 + nh - 1) / group - c_lo + 1;
    const PmMixLayout L = pm_mix_layout(hq, dv, p.ncv_mix, NK, HB);
    float* sc = reinterpret_cast<float*>(pm_smem + L.sc);
    bf16* sV = reinterpret_cast<bf16*>(pm_smem + L.v);
    bf16* pp = reinterpret_cast<bf16*>(pm_smem + L.pp);
    float* s_m = reinterpret_cast<float*>(pm_smem + L.m);
    float* s_il = reinterpret_cast<float*>(pm_smem + L.il);
    float* s_talk = reinterpret_cast<float*>(pm_smem + L.talk);
    int* s_cnt = reinterpret_cast<int*>(pm_smem + L.ints);
    int* s_first = s_cnt + PM_ROWS;
    int* s_nb = s_first + PM_ROWS;
    constexpr int LDC = NK + 4;                           // 16-byte rows for the copies; the mix reads along a row
    const int ldv = dv + PM_PAD, ldp = NK + PM_PAD;
    const int wide = d + dv;
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);

    if (tid < PM_ROWS) {
        int c = tid < nq ? p.row_count[r0 + tid] : 0;
        c = max(c, 0);
        const bool past = p.window > 0 && c > p.window;
        s_cnt[tid] = c;
        s_first[tid] = past ? c - p.window : 0;
        s_nb[tid] = (past && p.pool > 0) ? min((c - p.window) / p.pool, p.max_blocks) : 0;
    }
    for (int i = tid; i < nh * HMAX; i += PM_THREADS) {
        const int h = h0 + i / HMAX, g = i % HMAX;
        s_talk[i] = g >= hq ? 0.f : (p.talk != nullptr ? p.talk[(size_t)h * hq + g] : (h == g ? 1.f : 0.f));
    }
    for (int i = tid; i < hq * PM_ROWS; i += PM_THREADS) {
        const int g = i / PM_ROWS, r = i - g * PM_ROWS;
        float m = 0.f, il = 0.f;
        if (r < nq) {
            const float* st = p.stats + ((size_t)(r0 + r) * hq + g) * 2;
            m = st[0];
            il = st[1] > 0.f ? 1.f / st[1] : 0.f;
        }
        s_m[i] = m;
        s_il[i] = il;
    }
    __syncthreads();
    int nb_max = 0, first_min = 0x7fffffff, c_max = 0;
    for (int i = 0; i < nq; ++i) {
        nb_max = max(nb_max, s_nb[i]);
        first_min = min(first_min, s_first[i]);
        c_max = max(c_max, s_cnt[i]);
    }
    const int n_keys = c_max > 0 ? nb_max + (c_max - first_min) : 0;
    const int slot = p.slots[entry];
    const float* pooled = p.pooled + (size_t)((slot > 0 && slot < p.n_slots) ? slot : 0) * p.slot_stride;
    const int* pages = p.block_table + (size_t)entry * p.table_width;

    constexpr int OT = (DVMAX / 16 + SPLIT - 1) / SPLIT;   // 16-wide value tiles a warp
    float o[2 * OT][4];
#pragma unroll
    for (int n = 0; n < 2 * OT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

    constexpr int TPK = PM_THREADS / NK;
    auto issue = [&](int j0, int buf) {
        // the step's scores: rows of NK floats, [hq * 16] of them
        const float* from = p.kept + ((size_t)t * p.kept_steps + j0 / 16) * hq * PM_ROWS * 16;
        float* to = sc + (size_t)buf * hq * PM_ROWS * LDC;
        for (int idx = tid; idx < hq * PM_ROWS * (NK / 4); idx += PM_THREADS) {
            const int row = idx / (NK / 4), ch = idx - row * (NK / 4);
            pm_cp_async16(to + (size_t)row * LDC + ch * 4, from + ((size_t)(ch >> 2) * hq * PM_ROWS + row) * 16 + (ch & 3) * 4);
        }
        const int jj = tid / TPK, sub = tid - jj * TPK;
        const int j = j0 + jj;
        bf16* vd = sV + (size_t)buf * p.ncv_mix * NK * ldv + (size_t)jj * ldv;
        long long row = -1;
        if (j >= nb_max && j < n_keys) {
            const int pos = first_min + (j - nb_max);
            const int lp = pos / p.page_size;
            const int page = lp < p.table_width ? pages[lp] : -1;
            if (page >= 0 && page < p.n_pages) row = (long long)page * hkv * p.page_size + (pos - lp * p.page_size);
        }
        if (row >= 0) {
            for (int cl = 0; cl < ncv; ++cl) {
                const bf16* src = p.v_table + (size_t)(row + (long long)(c_lo + cl) * p.page_size) * dv;
                for (int ch = sub; ch * 8 < dv; ch += TPK) pm_cp_async16(vd + (size_t)cl * NK * ldv + ch * 8, src + ch * 8);
            }
        } else if (j < nb_max) {
            for (int cl = 0; cl < ncv; ++cl) {
                const float* src = pooled + ((size_t)j * hkv + c_lo + cl) * wide + d;
                for (int ch = sub; ch * 8 < dv; ch += TPK) {
                    const float4 a = *reinterpret_cast<const float4*>(src + ch * 8), b = *reinterpret_cast<const float4*>(src + ch * 8 + 4);
                    *reinterpret_cast<uint4*>(vd + (size_t)cl * NK * ldv + ch * 8) = make_uint4(pm_pack(a.x, a.y), pm_pack(a.z, a.w), pm_pack(b.x, b.y), pm_pack(b.z, b.w));
                }
            }
        } else {
            for (int cl = 0; cl < ncv; ++cl)
                for (int ch = sub; ch * 8 < dv; ch += TPK) *reinterpret_cast<uint4*>(vd + (size_t)cl * NK * ldv + ch * 8) = zero4;
        }
        pm_cp_async_commit();
    };

    if (n_keys > 0) issue(0, 0);
    for (int j0 = 0; j0 < n_keys; j0 += NK) {
        const int buf = (j0 / NK) & 1;
        pm_cp_async_wait_all();
        __syncthreads();                                     // the step's scores and values are in; everyone has left the step before
        if (j0 + NK < n_keys) issue(j0 + NK, buf ^ 1);
        const float* bS = sc + (size_t)buf * hq * PM_ROWS * LDC;
        const bf16* bV = sV + (size_t)buf * p.ncv_mix * NK * ldv;
        // a (token, key) pair a thread, or two threads that share its output heads when a step has fewer pairs than threads
        constexpr int EPT = PM_THREADS / (PM_ROWS * NK) > 0 ? PM_THREADS / (PM_ROWS * NK) : 1;
        for (int e = tid % (PM_ROWS * NK); e < PM_ROWS * NK; e += PM_THREADS) {
            const int i = e / NK, jj = e - i * NK;
            const int part = tid / (PM_ROWS * NK);
            float pg[HMAX];
#pragma unroll
            for (int g = 0; g < HMAX; ++g) {
                pg[g] = 0.f;
                if (g < hq) {
                    const float v = bS[(size_t)(g * PM_ROWS + i) * LDC + jj];
                    pg[g] = v == -INFINITY ? 0.f : __expf(v - s_m[g * PM_ROWS + i]) * s_il[g * PM_ROWS + i];
                }
            }
            for (int hl = part; hl < nh; hl += EPT) {
                const float4* tr = reinterpret_cast<const float4*>(s_talk + hl * HMAX);
                float w = 0.f;
#pragma unroll
                for (int g4 = 0; g4 < HMAX / 4; ++g4) {
                    const float4 t4 = tr[g4];
                    w = fmaf(t4.x, pg[4 * g4], w); w = fmaf(t4.y, pg[4 * g4 + 1], w);
                    w = fmaf(t4.z, pg[4 * g4 + 2], w); w = fmaf(t4.w, pg[4 * g4 + 3], w);
                }
                pp[(size_t)(hl * PM_ROWS + i) * ldp + jj] = __float2bfloat16(w);
            }
        }
        __syncthreads();
        if (warp < SPLIT * nh) {
            const int hl = warp / SPLIT, half = warp % SPLIT;
            const int cl = (h0 + hl) / group - c_lo;
            const bf16* pa = pp + (size_t)(hl * PM_ROWS + (lane & 15)) * ldp + (lane >> 4) * 8;
            const bf16* vf = bV + ((size_t)cl * NK + (lane & 7) + ((lane >> 3) & 1) * 8) * ldv + (lane >> 4) * 8 + half * OT * 16;
#pragma unroll
            for (int kk = 0; kk < NK; kk += 16) {
                uint32_t a[4];
                pm_ldmatrix_x4(a, pa + kk);
#pragma unroll
                for (int n2 = 0; n2 < OT; ++n2) {
                    if ((half * OT + n2) * 16 < dv) {
                        uint32_t b[4];
                        pm_ldmatrix_x4_trans(b, vf + (size_t)kk * ldv + n2 * 16);
                        pm_mma(o[2 * n2], a, b[0], b[1]);
                        pm_mma(o[2 * n2 + 1], a, b[2], b[3]);
                    }
                }
            }
        }
        // (the next step's first barrier stands between these reads of pp and its writes)
    }
    if (warp < SPLIT * nh) {
        const int h = h0 + warp / SPLIT, half = warp % SPLIT;
#pragma unroll
        for (int n = 0; n < 2 * OT; ++n) {
            const int col = (half * OT * 2 + n) * 8 + (lane & 3) * 2;
            if (col < dv) {
                const int i = lane >> 2;
                if (i < nq) *reinterpret_cast<uint32_t*>(p.out + ((size_t)(r0 + i) * hq + h) * dv + col) = pm_pack(o[n][0], o[n][1]);
                if (i + 8 < nq) *reinterpret_cast<uint32_t*>(p.out + ((size_t)(r0 + i + 8) * hq + h) * dv + col) = pm_pack(o[n][2], o[n][3]);
            }
        }
    }
}

// The most kv heads whose values any block of PM_HEADS output heads reads.
static int pm_value_heads(int hq, int hkv, int hb = PM_HEADS) {
    const int group = hq / hkv;
    int most = 1;
    for (int h0 = 0; h0 < hq; h0 += hb) {
        const int last = (h0 + hb < hq ? h0 + hb : hq) - 1;
        const int n = last / group - h0 / group + 1;
        if (n > most) most = n;
    }
    return most;
}

constexpr unsigned PM_SMEM_LIMIT = 227 * 1024;

// Output heads a block of the launch that reads kept scores.
static int pm_mix_heads(int hq) { return hq > PM_HEADS ? 16 : 8; }

// How the kernel runs these sizes: keys a step * 4 + stages, the first of (32, 2), (16, 2), (32, 1), (16, 1)
// that fits shared memory; 0 if the kernel does not take the sizes.
static int pm_form(int hq, int hkv, int d, int dv) {
    if (hq <= 0 || hkv <= 0 || hq % hkv != 0 || hq > 32 || d <= 0 || dv <= 0 || d % 16 != 0 || dv % 16 != 0 || dv > 128) return 0;
    const int ncv = pm_value_heads(hq, hkv);
    const int forms[4][2] = {{32, 2}, {16, 2}, {32, 1}, {16, 1}};
    for (const auto& f : forms)
        if (pm_layout(hq, hkv, d, dv, ncv, f[0], f[1]).total <= PM_SMEM_LIMIT) return f[0] * 4 + f[1];
    return 0;
}

template <int NK, int HMAX, int DVMAX, int STAGES>
static int pm_launch(PooledMmaParams p, int tiles, cudaStream_t s) {
    const unsigned smem = pm_layout(p.hq, p.hkv, p.d, p.dv, p.ncv, NK, STAGES).total;
    if (smem > 48 * 1024) cudaFuncSetAttribute(pooled_mma_kernel<NK, HMAX, DVMAX, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    p.mode = 1;
    pooled_mma_kernel<NK, HMAX, DVMAX, STAGES><<<dim3(tiles, 1), PM_THREADS, smem, s>>>(p);
    if (int e = check_launch("pooled_attention_mma statistics")) return e;
    p.mode = 2;
    pooled_mma_kernel<NK, HMAX, DVMAX, STAGES><<<dim3(tiles, (p.hq + PM_HEADS - 1) / PM_HEADS), PM_THREADS, smem, s>>>(p);
    return check_launch("pooled_attention_mma");
}

template <int NK, int HMAX, int STAGES>
static int pm_by_values(const PooledMmaParams& p, int tiles, cudaStream_t s) {
    return p.dv <= 64 ? pm_launch<NK, HMAX, 64, STAGES>(p, tiles, s) : pm_launch<NK, HMAX, 128, STAGES>(p, tiles, s);
}

template <int NK, int STAGES>
static int pm_by_heads(const PooledMmaParams& p, int tiles, cudaStream_t s) {
    if (p.hq <= 8) return pm_by_values<NK, 8, STAGES>(p, tiles, s);
    if (p.hq <= 16) return pm_by_values<NK, 16, STAGES>(p, tiles, s);
    return pm_by_values<NK, 32, STAGES>(p, tiles, s);
}

// ---- with kept scores: the statistics launch by blocks of heads, then the mix launch
static int pm_mix_keys(int hq, int hkv, int dv) {           // keys a step of the mix launch: 32, 16 or 0 (does not fit)
    const int hb = pm_mix_heads(hq), ncv = pm_value_heads(hq, hkv, hb);
    if (pm_mix_layout(hq, dv, ncv, 32, hb).total <= PM_SMEM_LIMIT) return 32;
    if (pm_mix_layout(hq, dv, ncv, 16, hb).total <= PM_SMEM_LIMIT) return 16;
    return 0;
}

static int pm_stats_form(int hq, int hkv, int d) {          // keys a step * 4 + stages of the statistics launch, or 0
    const int ncv = pm_value_heads(hq, hkv);
    const int forms[4][2] = {{32, 2}, {16, 2}, {32, 1}, {16, 1}};
    for (const auto& f : forms)
        if (pm_stats_layout(hq, d, ncv, f[0], f[1]).total <= PM_SMEM_LIMIT) return f[0] * 4 + f[1];
    return 0;
}

template <int NK, int STAGES>
static int pm_launch_stats(const PooledMmaParams& p, int tiles, cudaStream_t s) {
    const unsigned smem = pm_stats_layout(p.hq, p.d, p.ncv, NK, STAGES).total;
    if (smem > 48 * 1024) cudaFuncSetAttribute(pooled_stats_kernel<NK, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    pooled_stats_kernel<NK, STAGES><<<dim3(tiles, (p.hq + PM_HEADS - 1) / PM_HEADS), PM_THREADS, smem, s>>>(p);
    return check_launch("pooled_attention_mma statistics");
}

template <int NK, int HMAX, int DVMAX, int HB>
static int pm_launch_mix(const PooledMmaParams& p, int tiles, cudaStream_t s) {
    const unsigned smem = pm_mix_layout(p.hq, p.dv, p.ncv_mix, NK, HB).total;
    if (smem > 48 * 1024) cudaFuncSetAttribute(pooled_mix_kernel<NK, HMAX, DVMAX, HB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    pooled_mix_kernel<NK, HMAX, DVMAX, HB><<<dim3(tiles, (p.hq + HB - 1) / HB), PM_THREADS, smem, s>>>(p);
    return check_launch("pooled_attention_mma mix");
}

template <int NK>
static int pm_mix_by_sizes(const PooledMmaParams& p, int tiles, cudaStream_t s) {
    if (p.hq <= 8) return p.dv <= 64 ? pm_launch_mix<NK, 8, 64, 8>(p, tiles, s) : pm_launch_mix<NK, 8, 128, 8>(p, tiles, s);
    if (p.hq <= 16) return p.dv <= 64 ? pm_launch_mix<NK, 16, 64, 16>(p, tiles, s) : pm_launch_mix<NK, 16, 128, 16>(p, tiles, s);
    return p.dv <= 64 ? pm_launch_mix<NK, 32, 64, 16>(p, tiles, s) : pm_launch_mix<NK, 32, 128, 16>(p, tiles, s);
}

static int pm_run_kept(const PooledMmaParams& p, int tiles, cudaStream_t s) {
    int e;
    switch (pm_stats_form(p.hq, p.hkv, p.d)) {
        case 32 * 4 + 2: e = pm_launch_stats<32, 2>(p, tiles, s); break;
        case 16 * 4 + 2: e = pm_launch_stats<16, 2>(p, tiles, s); break;
        case 32 * 4 + 1: e = pm_launch_stats<32, 1>(p, tiles, s); break;
        default: e = pm_launch_stats<16, 1>(p, tiles, s); break;
    }
    if (e) return e;
    return pm_mix_keys(p.hq, p.hkv, p.dv) == 32 ? pm_mix_by_sizes<32>(p, tiles, s) : pm_mix_by_sizes<16>(p, tiles, s);
}

}  // namespace kb

using namespace kb;

// 1 if the tensor-core kernel takes these sizes (bfloat16 only), else 0.
extern "C" int kb_pooled_attention_mma_takes(int hq, int hkv, int d, int dv) { return pm_form(hq, hkv, d, dv) > 0 ? 1 : 0; }

extern "C" int kb_pooled_attention_mma_tile_rows() { return PM_ROWS; }

extern "C" long long kb_pooled_attention_mma_scratch_floats(int rows, int hq) { return (long long)rows * hq * 2; }

// Steps a tile needs room for when the first launch keeps its scores for the second: the most keys a tile of a
// request that has seen `longest` positions reads, over the keys a step.
static int pm_kept_steps(int window, int pool, int max_blocks, int longest) {      // runs of 16 keys, an even number
    long long tokens = window > 0 ? (longest < window + PM_ROWS - 1 ? longest : window + PM_ROWS - 1) : longest;
    long long blocks = (window > 0 && pool > 0 && longest > window) ? (longest - window) / pool : 0;
    if (blocks > max_blocks) blocks = max_blocks;
    return (int)((tokens + blocks + 31) / 32) * 2;
}

// Floats of scratch memory for the kept scores (0: these sizes are not taken).
extern "C" long long kb_pooled_attention_mma_kept_floats(int tiles, int hq, int hkv, int d, int dv, int window, int pool, int max_blocks,
                                                         int longest) {
    const int form = pm_form(hq, hkv, d, dv);
    if (form <= 0 || tiles <= 0 || longest <= 0) return 0;
    if (pm_mix_keys(hq, hkv, dv) == 0 || pm_stats_form(hq, hkv, d) == 0) return 0;
    return (long long)tiles * pm_kept_steps(window, pool, pool > 0 ? max_blocks : 0, longest) * hq * PM_ROWS * 16;
}

extern "C" int kb_pooled_attention_mma(void* out, const void* q, const void* k_table, const void* v_table, const float* pooled,
                                       long long slot_stride, int n_slots, int max_blocks, const int* block_table,
                                       const int* row_count, const int* tile_entry, const int* tile_row0, const int* tile_nq,
                                       int tiles, const int* slots, const float* talk, const float* temp, int rows, int hq, int hkv,
                                       int d, int dv, int page_size, int table_width, int n_pages, int window, int pool, float scale,
                                       float* scratch, float* kept, int longest, void* stream) {
    KB_REQUIRE(rows >= 0 && tiles >= 0 && hq > 0 && hkv > 0 && hq % hkv == 0, "pooled_attention_mma: rows %d, tiles %d, %d heads over %d", rows, tiles, hq, hkv);
    const int form = pm_form(hq, hkv, d, dv);
    KB_REQUIRE(form > 0, "pooled_attention_mma: %d heads over %d of sizes %d / %d are not taken", hq, hkv, d, dv);
    KB_REQUIRE(page_size > 0 && table_width > 0 && n_pages > 0, "pooled_attention_mma: page_size %d, table width %d, pages %d", page_size, table_width, n_pages);
    KB_REQUIRE(window >= 0 && pool >= 0 && max_blocks >= 0, "pooled_attention_mma: window %d, blocks of %d, %d blocks", window, pool, max_blocks);
    KB_REQUIRE(pool == 0 || (pooled != nullptr && n_slots > 0 && slot_stride >= (long long)max_blocks * hkv * (d + dv) && slot_stride % 4 == 0),
               "pooled_attention_mma: blocks of %d without a table that holds %d of them a slot", pool, max_blocks);
    KB_REQUIRE(scratch != nullptr && tile_entry != nullptr && tile_row0 != nullptr && tile_nq != nullptr, "pooled_attention_mma: no tiles or no scratch memory");
    if (rows == 0 || tiles == 0) return 0;
    PooledMmaParams p;
    p.q = (const bf16*)q; p.k_table = (const bf16*)k_table; p.v_table = (const bf16*)v_table; p.pooled = pooled;
    p.block_table = block_table; p.row_count = row_count; p.tile_entry = tile_entry; p.tile_row0 = tile_row0; p.tile_nq = tile_nq;
    p.slots = slots; p.talk = talk; p.temp = temp; p.out = (bf16*)out; p.stats = scratch; p.slot_stride = slot_stride;
    p.hq = hq; p.hkv = hkv; p.d = d; p.dv = dv; p.page_size = page_size; p.table_width = table_width; p.n_pages = n_pages;
    p.n_slots = n_slots; p.max_blocks = pool > 0 ? max_blocks : 0; p.window = window; p.pool = pool; p.ncv = pm_value_heads(hq, hkv);
    p.mode = 1; p.scale = scale;
    p.ncv_mix = pm_value_heads(hq, hkv, pm_mix_heads(hq));
    p.kept = kept;                                          // sized by kb_pooled_attention_mma_kept_floats for the same `longest`
    p.kept_steps = kept != nullptr ? pm_kept_steps(window, pool, p.max_blocks, longest) : 0;
    KB_REQUIRE(kept == nullptr || longest > 0, "pooled_attention_mma: kept scores without the longest request's positions");
    cudaStream_t s = (cudaStream_t)stream;
    if (kept != nullptr) return pm_run_kept(p, tiles, s);
    switch (form) {
        case 32 * 4 + 2: return pm_by_heads<32, 2>(p, tiles, s);
        case 16 * 4 + 2: return pm_by_heads<16, 2>(p, tiles, s);
        case 32 * 4 + 1: return pm_by_heads<32, 1>(p, tiles, s);
        default: return pm_by_heads<16, 1>(p, tiles, s);
    }
}
