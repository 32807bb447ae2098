// The C entry points of paged attention; the kernels are in attention_rows.cuh.
#include "attention_rows.cuh"

using namespace kb;

extern "C" int kb_attention_chunk() { return ATT_CHUNK; }

// Scratch floats for `slots` chunk slots (0 when slots == 1).
extern "C" long long kb_paged_attention_scratch_floats(int rows, int hq, int d, int slots) {
    return slots > 1 ? (long long)rows * hq * slots * (d + 2) : 0;      // d: the values' size
}

extern "C" int kb_paged_attention_rows_blocked(void* out, const void* q, const void* k_table, const void* v_table, int dt,
                                       const int* block_table, const int* row_entry, const int* row_count, int rows,
                                       int hq, int hkv, int d, int dv, int page_size, int table_width, int n_pages, int window,
                                       int keep, int slots, float scale, float cap, float* scratch, int v_stride, const float* sinks,
                                       int block, void* stream) {
    KB_REQUIRE(rows >= 0 && hq > 0 && hkv > 0 && hq % hkv == 0, "paged_attention: rows %d, heads %d over %d kv heads", rows, hq, hkv);
    KB_REQUIRE(d > 0 && dv > 0, "paged_attention: head sizes %d / %d", d, dv);
    KB_REQUIRE(v_stride >= dv, "paged_attention: values of %d lie %d apart", dv, v_stride);
    KB_REQUIRE(keep >= 0, "paged_attention: %d first keys kept", keep);
    KB_REQUIRE(block >= 0 && (block == 0 || keep == 0), "paged_attention: blocks of %d positions with %d first keys kept", block, keep);
    KB_REQUIRE(page_size > 0 && table_width > 0 && n_pages > 0, "paged_attention: page_size %d, table width %d, pages %d", page_size, table_width, n_pages);
    KB_REQUIRE(window >= 0 && slots >= 1 && slots <= 65535, "paged_attention: window %d, chunk slots %d", window, slots);
    KB_REQUIRE(cap >= 0.f, "paged_attention: cap %g is negative", cap);
    KB_REQUIRE(slots == 1 || scratch != nullptr, "paged_attention: %d chunk slots need scratch memory", slots);
    KB_REQUIRE(rows <= 0x7fffffff / 1 && (long long)hkv * ((hq / hkv + 7) / 8) <= 65535, "paged_attention: too many heads for one launch");
    if (rows == 0) return 0;
    AttParams p;
    p.q = q; p.k_table = k_table; p.v_table = v_table; p.block_table = block_table; p.row_entry = row_entry;
    p.row_count = row_count; p.out = out; p.partial = slots > 1 ? scratch : nullptr;
    p.rows = rows; p.hq = hq; p.hkv = hkv; p.d = d; p.page_size = page_size; p.table_width = table_width;
    p.n_pages = n_pages; p.dv = dv; p.vec = (d % (dt == KB_DT_F32 ? 4 : 8)) == 0 && ((uintptr_t)k_table & 15) == 0; p.window = window; p.keep = window > 0 ? keep : 0;
    p.keep_slots = p.keep > 0 ? (p.keep + ATT_CHUNK - 1) / ATT_CHUNK : 0;
    KB_REQUIRE(slots > p.keep_slots, "paged_attention: %d slots of which %d are the kept first keys'", slots, p.keep_slots);
    p.slots = slots; p.chunk = ATT_CHUNK; p.scale = scale; p.cap = cap; p.v_stride = v_stride; p.sinks = sinks; p.block = block;
    cudaStream_t s = (cudaStream_t)stream;
    if (dt == KB_DT_F32) return rows_f32(p, s, slots > 1);
    if (dt == KB_DT_BF16) return rows_bf16(p, s, slots > 1);
    return fail("paged_attention: dtype code %d is not known", dt);
}

extern "C" int kb_paged_attention_rows(void* out, const void* q, const void* k_table, const void* v_table, int dt,
                                       const int* block_table, const int* row_entry, const int* row_count, int rows,
                                       int hq, int hkv, int d, int dv, int page_size, int table_width, int n_pages, int window,
                                       int keep, int slots, float scale, float cap, float* scratch, int v_stride, const float* sinks,
                                       void* stream) {
    return kb_paged_attention_rows_blocked(out, q, k_table, v_table, dt, block_table, row_entry, row_count, rows, hq, hkv, d, dv, page_size,
                                           table_width, n_pages, window, keep, slots, scale, cap, scratch, v_stride, sinks, 0, stream);
}
