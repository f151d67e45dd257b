// `.vib3` container for INT4 expert pages: quantiser, page-split writer and reader (host side, no CUDA).
//
// What it follows in the reference:
//   quantiser      quantize_weights_to_int4, src/compute/kernels.rs:3778-3831 (group 32, scale = max|w| / 7,
//                  q = clamp(round(w / scale) + 8, 0, 15), low nibble = even column; the reference stores the
//                  scale as bf16, its CUDA kernels decode fp16: the caller picks the encoding)
//   page split     add_pages_from_data, src/storage/convert.rs:1841-1901 (rows_per_page = 2 MiB / bytes_per_row,
//                  a page = its rows' codes followed by its rows' scales)
//   file layout    Vib3Header (512 bytes), metadata JSON, PageCatalogEntry (48 bytes) sorted by (layer, expert,
//                  segment, page), ExpertIndexEntry (20 bytes), page data from a 2 MiB boundary with every page
//                  on a 4096-byte boundary: src/storage/format.rs:50-141, :146-154, :842-1090
//   reader         Vib3File::open, src/storage/format.rs:241-339 (magic, version, section bounds)
// Only uncompressed pages are written and read (compression code 0); the vector index, co-activation table and
// materialised views of the format are written empty.
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <cmath>
#include <map>
#include <new>
#include <string>
#include <vector>

#include "page_pool.hpp"
#include "vib3_b200.h"

namespace {

constexpr uint64_t kMagic = 0x3342495600000001ull;   // format.rs:39
constexpr uint32_t kVersion = 1;
constexpr size_t kHeaderSize = 512;
constexpr size_t kPageSize = 2u << 20;
constexpr int kGroup = 32;

#pragma pack(push, 1)
struct Header {   // format.rs:50-92
    uint64_t magic;
    uint32_t version, flags;
    uint64_t metadata_offset, metadata_size;
    uint64_t page_catalog_offset, page_catalog_size;
    uint32_t page_catalog_count;
    uint64_t expert_index_offset, expert_index_size;
    uint64_t vector_index_offset, vector_index_size;
    uint64_t coactivation_offset, coactivation_size;
    uint64_t view_catalog_offset, view_catalog_size;
    uint32_t view_count;
    uint64_t page_data_offset, page_data_size;
    uint32_t num_layers, num_experts, num_active_experts, hidden_dim, expert_hidden_dim;
    uint8_t expert_dtype, shared_dtype;
    uint8_t reserved[354];
};
struct CatalogEntry {   // format.rs:100-124
    uint16_t layer, expert, segment, page_idx;
    uint64_t file_offset;
    uint32_t compressed_size, raw_size;
    uint16_t row_start, row_count, col_start, col_count;
    float mean_activation, access_frequency;
    uint16_t coactivation_cluster;
    uint8_t compression, flags;
    uint8_t pad[4];
};
struct ExpertIndexEntry {   // format.rs:146-154
    uint16_t layer, expert;
    uint32_t first_page_idx, page_count, total_bytes;
    uint16_t num_segments, reserved;
};
#pragma pack(pop)
static_assert(sizeof(Header) == kHeaderSize, "header is 512 bytes");
static_assert(sizeof(CatalogEntry) == 48, "catalog entry is 48 bytes");
static_assert(sizeof(ExpertIndexEntry) == 20, "expert index entry is 20 bytes");

uint16_t f32_to_bf16(float f) {   // round to nearest even (crate `half`)
    uint32_t b;
    memcpy(&b, &f, 4);
    if ((b & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((b >> 16) | 0x40);
    const uint32_t r = 0x7FFFu + ((b >> 16) & 1u);
    return (uint16_t)((b + r) >> 16);
}

uint16_t f32_to_f16(float f) {   // round to nearest even, overflow to infinity, subnormals
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const uint32_t e = (x >> 23) & 0xFFu, m = x & 0x7FFFFFu;
    if (e == 0xFF) return (uint16_t)(sign | 0x7C00u | (m ? 0x200u | (m >> 13) : 0));
    const int ex = (int)e - 127 + 15;
    if (ex >= 31) return (uint16_t)(sign | 0x7C00u);
    if (ex <= 0) {
        if (ex < -10) return (uint16_t)sign;
        const uint32_t mant = m | 0x800000u;
        const int shift = 14 - ex;
        uint32_t h = mant >> shift;
        const uint32_t rem = mant & ((1u << shift) - 1), half = 1u << (shift - 1);
        if (rem > half || (rem == half && (h & 1))) ++h;
        return (uint16_t)(sign | h);
    }
    uint32_t h = ((uint32_t)ex << 10) | (m >> 13);
    const uint32_t rem = m & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1))) ++h;
    return (uint16_t)(sign | h);
}

struct PendingPage {
    CatalogEntry entry;
    std::vector<uint8_t> data;
};

}  // namespace

struct vib3_writer {
    std::string path, metadata;
    Header head;
    std::vector<PendingPage> pages;
};

struct vib3_file {
    std::vector<uint8_t> meta;
    std::vector<CatalogEntry> catalog;
    std::vector<ExpertIndexEntry> experts;
    Header head;
    FILE* f = nullptr;
};

extern "C" size_t vib3_int4_matrix_bytes(int rows, int cols) {
    if (rows <= 0 || cols <= 0) return 0;
    return (size_t)rows * ((cols + 1) / 2) + (size_t)rows * ((cols + kGroup - 1) / kGroup) * 2;
}

// out: [rows][ceil(cols / 2)] code bytes, then [rows][ceil(cols / 32)] 16-bit scales.  scale_format 0 = bf16 (what
// the reference's quantiser writes), 1 = fp16 (what its CUDA kernels and this library's kernels decode).
extern "C" int vib3_quantize_int4(const float* w, int rows, int cols, int scale_format, uint8_t* out) {
    if (!w || !out) return VIB3_ERR_NULL;
    if (rows <= 0 || cols <= 0) return VIB3_ERR_SHAPE;
    if (scale_format != 0 && scale_format != 1) return VIB3_ERR_UNSUPPORTED;
    const size_t packed_k = (size_t)(cols + 1) / 2, groups = (size_t)(cols + kGroup - 1) / kGroup;
    uint8_t* codes = out;
    uint8_t* scales = out + (size_t)rows * packed_k;
    memset(out, 0, (size_t)rows * packed_k);
    for (int r = 0; r < rows; ++r) {
        const float* row = w + (size_t)r * cols;
        for (size_t g = 0; g < groups; ++g) {
            const int c0 = (int)g * kGroup, c1 = std::min(c0 + kGroup, cols);
            float mx = 0.f;
            for (int c = c0; c < c1; ++c) mx = std::fmax(mx, std::fabs(row[c]));
            const float scale = mx > 0.f ? mx / 7.0f : 1.0f;
            const uint16_t sb = scale_format == 0 ? f32_to_bf16(scale) : f32_to_f16(scale);
            scales[((size_t)r * groups + g) * 2] = (uint8_t)(sb & 0xFF);
            scales[((size_t)r * groups + g) * 2 + 1] = (uint8_t)(sb >> 8);
            for (int c = c0; c < c1; ++c) {
                // Rust's f32::round: half away from zero
                int q = (int)std::round(row[c] / scale) + 8;
                q = std::min(15, std::max(0, q));
                codes[(size_t)r * packed_k + c / 2] |= (uint8_t)((c & 1) ? (q & 0xF) << 4 : (q & 0xF));
            }
        }
    }
    return VIB3_OK;
}

extern "C" vib3_writer* vib3_writer_create(const char* path, const char* metadata_json, uint32_t num_layers, uint32_t num_experts,
                                           uint32_t num_active_experts, uint32_t hidden_dim, uint32_t expert_hidden_dim) {
    if (!path) return nullptr;
    vib3_writer* w = new (std::nothrow) vib3_writer();
    if (!w) return nullptr;
    w->path = path;
    w->metadata = metadata_json ? metadata_json : "{}";
    memset(&w->head, 0, sizeof(Header));
    w->head.magic = kMagic;
    w->head.version = kVersion;
    w->head.num_layers = num_layers;
    w->head.num_experts = num_experts;
    w->head.num_active_experts = num_active_experts;
    w->head.hidden_dim = hidden_dim;
    w->head.expert_hidden_dim = expert_hidden_dim;
    w->head.expert_dtype = 5;   // DType::INT4, src/core/types.rs:633-642
    w->head.shared_dtype = 5;
    return w;
}

extern "C" void vib3_writer_destroy(vib3_writer* w) { delete w; }

// Cut a quantised matrix (the layout vib3_quantize_int4 writes) into pages and queue them; returns the number of
// pages, or VIB3_ERR_*.
extern "C" int vib3_writer_add_int4_matrix(vib3_writer* w, uint16_t layer, uint16_t expert, uint16_t segment, int rows, int cols,
                                           const uint8_t* int4_data) {
    if (!w || !int4_data) return VIB3_ERR_NULL;
    if (rows <= 0 || cols <= 0 || rows > 65535 || cols > 65535) return VIB3_ERR_SHAPE;
    const size_t packed_k = (size_t)(cols + 1) / 2, groups = (size_t)(cols + kGroup - 1) / kGroup;
    const size_t bytes_per_row = packed_k + groups * 2;
    const size_t rows_per_page = std::max<size_t>(kPageSize / bytes_per_row, 1);
    const size_t num_pages = ((size_t)rows + rows_per_page - 1) / rows_per_page;
    if (num_pages > 65535) return VIB3_ERR_COUNT;
    const uint8_t* scales = int4_data + (size_t)rows * packed_k;
    for (size_t p = 0; p < num_pages; ++p) {
        const size_t r0 = p * rows_per_page, rc = std::min(rows_per_page, (size_t)rows - r0);
        PendingPage pg;
        pg.data.resize(rc * bytes_per_row);
        memcpy(pg.data.data(), int4_data + r0 * packed_k, rc * packed_k);
        memcpy(pg.data.data() + rc * packed_k, scales + r0 * groups * 2, rc * groups * 2);
        memset(&pg.entry, 0, sizeof(CatalogEntry));
        pg.entry.layer = layer; pg.entry.expert = expert; pg.entry.segment = segment; pg.entry.page_idx = (uint16_t)p;
        pg.entry.compressed_size = pg.entry.raw_size = (uint32_t)pg.data.size();
        pg.entry.row_start = (uint16_t)r0; pg.entry.row_count = (uint16_t)rc; pg.entry.col_count = (uint16_t)cols;
        w->pages.push_back(std::move(pg));
    }
    return (int)num_pages;
}

extern "C" int vib3_writer_finalize(vib3_writer* w) {
    if (!w) return VIB3_ERR_NULL;
    // catalog order: (layer, expert, segment, page) — format.rs:881-892
    std::vector<size_t> order(w->pages.size());
    for (size_t i = 0; i < order.size(); ++i) order[i] = i;
    std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) {
        const CatalogEntry &x = w->pages[a].entry, &y = w->pages[b].entry;
        if (x.layer != y.layer) return x.layer < y.layer;
        if (x.expert != y.expert) return x.expert < y.expert;
        if (x.segment != y.segment) return x.segment < y.segment;
        return x.page_idx < y.page_idx;
    });
    std::vector<ExpertIndexEntry> experts;
    for (size_t i = 0; i < order.size();) {
        const CatalogEntry& e = w->pages[order[i]].entry;
        ExpertIndexEntry x;
        memset(&x, 0, sizeof(x));
        x.layer = e.layer; x.expert = e.expert; x.first_page_idx = (uint32_t)i;
        std::vector<uint16_t> segs;
        size_t j = i;
        for (; j < order.size(); ++j) {
            const CatalogEntry& f = w->pages[order[j]].entry;
            if (f.layer != e.layer || f.expert != e.expert) break;
            x.total_bytes += f.raw_size;
            if (std::find(segs.begin(), segs.end(), f.segment) == segs.end()) segs.push_back(f.segment);
        }
        x.page_count = (uint32_t)(j - i);
        x.num_segments = (uint16_t)segs.size();
        experts.push_back(x);
        i = j;
    }
    Header& h = w->head;
    h.metadata_offset = kHeaderSize;
    h.metadata_size = w->metadata.size();
    h.page_catalog_offset = h.metadata_offset + h.metadata_size;
    h.page_catalog_count = (uint32_t)order.size();
    h.page_catalog_size = (uint64_t)order.size() * sizeof(CatalogEntry);
    h.expert_index_offset = h.page_catalog_offset + h.page_catalog_size;
    h.expert_index_size = (uint64_t)experts.size() * sizeof(ExpertIndexEntry);
    h.vector_index_offset = h.expert_index_offset + h.expert_index_size;
    h.coactivation_offset = h.vector_index_offset;
    h.view_catalog_offset = h.coactivation_offset;
    h.page_data_offset = (h.view_catalog_offset + kPageSize - 1) / kPageSize * kPageSize;
    uint64_t off = h.page_data_offset;
    for (size_t i : order) {
        w->pages[i].entry.file_offset = off;
        off += ((uint64_t)w->pages[i].data.size() + 4095) / 4096 * 4096;
    }
    h.page_data_size = off - h.page_data_offset;
    FILE* f = fopen(w->path.c_str(), "wb");
    if (!f) return VIB3_ERR_STATE;
    bool ok = fwrite(&h, sizeof(Header), 1, f) == 1;
    ok = ok && (w->metadata.empty() || fwrite(w->metadata.data(), w->metadata.size(), 1, f) == 1);
    for (size_t i : order) ok = ok && fwrite(&w->pages[i].entry, sizeof(CatalogEntry), 1, f) == 1;
    for (const ExpertIndexEntry& x : experts) ok = ok && fwrite(&x, sizeof(x), 1, f) == 1;
    std::vector<uint8_t> zeros(4096, 0);
    for (size_t i : order) {
        const PendingPage& pg = w->pages[i];
        ok = ok && fseek(f, (long)pg.entry.file_offset, SEEK_SET) == 0;
        ok = ok && fwrite(pg.data.data(), pg.data.size(), 1, f) == 1;
        const size_t padn = (4096 - pg.data.size() % 4096) % 4096;
        ok = ok && (padn == 0 || fwrite(zeros.data(), padn, 1, f) == 1);
    }
    ok = fclose(f) == 0 && ok;
    return ok ? VIB3_OK : VIB3_ERR_STATE;
}

extern "C" vib3_file* vib3_file_open(const char* path, int* error_out) {
    auto fail = [&](int code, vib3_file* v) -> vib3_file* {
        if (error_out) *error_out = code;
        if (v && v->f) fclose(v->f);
        delete v;
        return nullptr;
    };
    if (!path) return fail(VIB3_ERR_NULL, nullptr);
    vib3_file* v = new (std::nothrow) vib3_file();
    if (!v) return fail(VIB3_ERR_STATE, nullptr);
    v->f = fopen(path, "rb");
    if (!v->f) return fail(VIB3_ERR_STATE, v);
    fseek(v->f, 0, SEEK_END);
    const uint64_t size = (uint64_t)ftell(v->f);
    fseek(v->f, 0, SEEK_SET);
    if (size < kHeaderSize || fread(&v->head, sizeof(Header), 1, v->f) != 1) return fail(VIB3_ERR_SHAPE, v);   // "file too small for header"
    if (v->head.magic != kMagic) return fail(VIB3_ERR_UNSUPPORTED, v);                                         // "bad magic"
    if (v->head.version != kVersion) return fail(VIB3_ERR_UNSUPPORTED, v);
    const Header& h = v->head;
    if (h.metadata_offset + h.metadata_size > size) return fail(VIB3_ERR_RANGE, v);
    if (h.page_catalog_offset + (uint64_t)h.page_catalog_count * sizeof(CatalogEntry) > size) return fail(VIB3_ERR_RANGE, v);
    v->meta.resize(h.metadata_size);
    fseek(v->f, (long)h.metadata_offset, SEEK_SET);
    if (h.metadata_size && fread(v->meta.data(), h.metadata_size, 1, v->f) != 1) return fail(VIB3_ERR_RANGE, v);
    v->catalog.resize(h.page_catalog_count);
    fseek(v->f, (long)h.page_catalog_offset, SEEK_SET);
    if (h.page_catalog_count && fread(v->catalog.data(), sizeof(CatalogEntry), h.page_catalog_count, v->f) != h.page_catalog_count)
        return fail(VIB3_ERR_RANGE, v);
    const uint64_t n_exp = h.expert_index_size / sizeof(ExpertIndexEntry);
    if (n_exp && h.expert_index_offset + h.expert_index_size <= size) {
        v->experts.resize(n_exp);
        fseek(v->f, (long)h.expert_index_offset, SEEK_SET);
        if (fread(v->experts.data(), sizeof(ExpertIndexEntry), n_exp, v->f) != n_exp) v->experts.clear();
    }
    for (const CatalogEntry& e : v->catalog)
        if (e.file_offset + e.compressed_size > size) return fail(VIB3_ERR_RANGE, v);
    if (error_out) *error_out = VIB3_OK;
    return v;
}

extern "C" void vib3_file_close(vib3_file* v) {
    if (!v) return;
    if (v->f) fclose(v->f);
    delete v;
}

extern "C" int vib3_file_page_count(const vib3_file* v) { return v ? (int)v->catalog.size() : VIB3_ERR_NULL; }

extern "C" int vib3_file_summary(const vib3_file* v, uint32_t* num_layers, uint32_t* num_experts, uint32_t* num_active_experts,
                                 uint32_t* hidden_dim, uint32_t* expert_hidden_dim, uint32_t* expert_dtype, uint64_t* page_data_offset) {
    if (!v) return VIB3_ERR_NULL;
    if (num_layers) *num_layers = v->head.num_layers;
    if (num_experts) *num_experts = v->head.num_experts;
    if (num_active_experts) *num_active_experts = v->head.num_active_experts;
    if (hidden_dim) *hidden_dim = v->head.hidden_dim;
    if (expert_hidden_dim) *expert_hidden_dim = v->head.expert_hidden_dim;
    if (expert_dtype) *expert_dtype = v->head.expert_dtype;
    if (page_data_offset) *page_data_offset = v->head.page_data_offset;
    return VIB3_OK;
}

extern "C" int vib3_file_page_info(const vib3_file* v, int index, vib3_file_page* out) {
    if (!v || !out) return VIB3_ERR_NULL;
    if (index < 0 || (size_t)index >= v->catalog.size()) return VIB3_ERR_RANGE;
    const CatalogEntry& e = v->catalog[index];
    out->layer = e.layer; out->expert = e.expert; out->segment = e.segment; out->page_idx = e.page_idx;
    out->row_start = e.row_start; out->row_count = e.row_count; out->col_count = e.col_count; out->compression = e.compression;
    out->file_offset = e.file_offset; out->raw_size = e.raw_size;
    return VIB3_OK;
}

extern "C" int vib3_file_read_page(vib3_file* v, int index, void* dst, size_t dst_bytes) {
    if (!v || !dst) return VIB3_ERR_NULL;
    if (index < 0 || (size_t)index >= v->catalog.size()) return VIB3_ERR_RANGE;
    const CatalogEntry& e = v->catalog[index];
    if (e.compression != 0) return VIB3_ERR_UNSUPPORTED;
    if (dst_bytes < e.raw_size) return VIB3_ERR_CAPACITY;
    if (fseek(v->f, (long)e.file_offset, SEEK_SET) != 0 || fread(dst, e.raw_size, 1, v->f) != 1) return VIB3_ERR_STATE;
    return VIB3_OK;
}

// Place every page of the file (of layers [layer_lo, layer_hi) and experts [expert_lo, expert_hi) or the shared
// expert 0xFFFF) into the pool — the role of PageBufferManager::preload_all (src/storage/buffer_manager.rs:1226-1254).
// Returns the number of pages loaded, or VIB3_ERR_*.
extern "C" long long vib3_file_load_into_pool(vib3_file* v, vib3_pool* pool, int layer_lo, int layer_hi, int expert_lo, int expert_hi) {
    if (!v || !pool) return VIB3_ERR_NULL;
    std::vector<uint8_t> buf(kPageSize);
    long long n = 0;
    for (size_t i = 0; i < v->catalog.size(); ++i) {
        const CatalogEntry& e = v->catalog[i];
        if (e.layer < layer_lo || e.layer >= layer_hi) continue;
        if (e.expert != 0xFFFF && (e.expert < expert_lo || e.expert >= expert_hi)) continue;
        if (e.raw_size > kPageSize) return VIB3_ERR_CAPACITY;
        if (int err = vib3_file_read_page(v, (int)i, buf.data(), buf.size())) return err;
        const long long slot = vib3_pool_load_page(pool, e.layer, e.expert, e.segment, e.page_idx, e.row_start, e.row_count, buf.data(), e.raw_size);
        if (slot < 0) return slot;
        ++n;
    }
    return n;
}
