// wpk.cu -- reader of the packed weight file (WPK v1) and loader into the B200 arena layout.
//
// File format (little-endian; tools/minicpm_common.py:47-75, 318-348; C++ mirror
// native/runtime/weight_loader.cpp:21-50): 64-byte header {magic "MKP1", abi_version 2,
// target_sm, model_hash[32], section_count, reserved 0, toc_offset 64, data_start},
// then section_count TOC entries of 132 packed bytes {name_hash (FNV-1a 64 of the
// section name), dtype (0 bf16, 2 e4m3 + fp32 row scales), layout 0, rank, dims[8],
// data_offset (256-byte aligned), data_bytes, scale_offset, scale_bytes, reserved[6]}.
// Validation follows native/runtime/weight_loader.cpp:225-330 (magic, version, TOC span,
// duplicate hashes, section bounds); files written for target_sm 120 are accepted: the
// payload is plain row-major and only the placement in device memory differs here.
// What is new: a section can be uploaded as an N-shard (a row range) and the fused
// gate_up section can be re-laid with gate and up rows interleaved on the way.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "common.cuh"

namespace mcl {

#pragma pack(push, 1)
struct WpkHeader {
    uint32_t magic;
    uint16_t abi_version, target_sm;
    uint8_t model_hash[32];
    uint32_t section_count, reserved;
    uint64_t toc_offset, data_start;
};
struct WpkToc {
    uint64_t name_hash;
    uint32_t dtype, layout, rank, dims[8];
    uint64_t data_offset, data_bytes, scale_offset, scale_bytes, reserved[6];
};
#pragma pack(pop)
static_assert(sizeof(WpkHeader) == 64 && sizeof(WpkToc) == 132, "packed WPK v1 records");

static uint64_t fnv1a64(const char* s) {
    uint64_t h = 0xCBF29CE484222325ull;
    for (; *s; ++s) h = (h ^ (uint8_t)*s) * 0x100000001B3ull;
    return h;
}


// ---- host-side quantiser of the packer -----------------------------------------------
// float -> e4m3 code with the packer's rule (tools/minicpm_common.py:130-171): round to nearest
// even on the 3-bit mantissa, magnitudes beyond 448 -- infinities and NaN included -- saturate
// to +/-448, the codes 0x7F / 0xFF are never produced.  Done in exact double arithmetic: the
// magnitude is put on the integer grid of its binade (2^(e-3), subnormal grid 2^-9) and rounded
// half to even there.
static uint8_t e4m3_from_f32(float f) {
    uint32_t bits;
    std::memcpy(&bits, &f, 4);
    const uint8_t sign = (uint8_t)((bits >> 31) << 7);
    double mag = std::fabs((double)f);
    if (!std::isfinite(mag)) mag = 1e9;
    int e = 0;
    (void)std::frexp(mag, &e);
    e -= 1;
    if (e < -6 || mag == 0.0) e = -6;
    const double step = std::ldexp(1.0, e - 3);
    double val = std::nearbyint(mag / step) * step;          // default rounding mode: half to even
    if (val > 448.0) val = 448.0;
    uint32_t code;
    if (val >= std::ldexp(1.0, -6)) {
        int e2 = 0;
        (void)std::frexp(val, &e2);
        e2 -= 1;
        code = ((uint32_t)(e2 + 7) << 3) + (uint32_t)(val / std::ldexp(1.0, e2) * 8.0 - 8.0);
    } else {
        code = (uint32_t)(val * 512.0);
    }
    if (code > 0x7Eu) code = 0x7Eu;
    return (uint8_t)(sign | code);
}

static float bf16_bits_to_f32(uint16_t b) {
    const uint32_t u = (uint32_t)b << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

}  // namespace mcl

using namespace mcl;

struct mc_sm100_wpk_writer {
    FILE* f;
    std::string path;
    WpkHeader hdr;
    std::vector<WpkToc> toc;
    uint32_t max_sections;
    uint64_t cursor;            // next free 256-byte aligned file offset
};

struct mc_sm100_wpk {
    FILE* f;
    uint64_t file_size;
    WpkHeader hdr;
    std::vector<WpkToc> toc;
};

static const WpkToc* find_section(const mc_sm100_wpk* h, const char* name) {
    const uint64_t key = fnv1a64(name);
    for (const auto& t : h->toc)
        if (t.name_hash == key) return &t;
    return nullptr;
}

extern "C" {

uint64_t mc_sm100_wpk_name_hash(const char* name) { return name ? fnv1a64(name) : 0; }

mc_status_t mc_sm100_wpk_open(const char* path, mc_sm100_wpk_t* out) {
    clear_error();
    if (out != nullptr) *out = nullptr;
    if (path == nullptr || out == nullptr) { set_error("mc_sm100_wpk_open: invalid args"); return MC_E_INVALID_ARGUMENT; }
    FILE* f = std::fopen(path, "rb");
    if (f == nullptr) { set_error("wpk: cannot open '%s'", path); return MC_E_IO; }
    mc_sm100_wpk* h = new (std::nothrow) mc_sm100_wpk();
    if (h == nullptr) { std::fclose(f); set_error("wpk: out of host memory"); return MC_E_OUT_OF_MEMORY; }
    h->f = f;
    auto fail = [&](mc_status_t st) { std::fclose(f); delete h; return st; };
    if (std::fseek(f, 0, SEEK_END) != 0) { set_error("wpk: seek failed"); return fail(MC_E_IO); }
    h->file_size = (uint64_t)std::ftell(f);
    if (h->file_size < sizeof(WpkHeader) || std::fseek(f, 0, SEEK_SET) != 0 ||
        std::fread(&h->hdr, sizeof(WpkHeader), 1, f) != 1) {
        set_error("wpk: file of %llu bytes has no header", (unsigned long long)h->file_size);
        return fail(MC_E_IO);
    }
    const WpkHeader& hd = h->hdr;
    if (hd.magic != 0x31504B4Du) { set_error("wpk magic mismatch: got 0x%08x expected 0x31504b4d", hd.magic); return fail(MC_E_MODEL_MISMATCH); }
    if (hd.abi_version != 2) { set_error("wpk abi_version mismatch: got 0x%04x expected 0x0002", hd.abi_version); return fail(MC_E_MODEL_MISMATCH); }
    if (hd.target_sm != 120 && hd.target_sm != 100) { set_error("wpk target_sm %u is neither 120 nor 100", hd.target_sm); return fail(MC_E_MODEL_MISMATCH); }
    if (hd.toc_offset != 64) { set_error("wpk toc_offset must be 64 (got %llu)", (unsigned long long)hd.toc_offset); return fail(MC_E_MODEL_MISMATCH); }
    if (hd.reserved != 0) { set_error("wpk reserved must be 0 (got %u)", hd.reserved); return fail(MC_E_MODEL_MISMATCH); }
    if (hd.data_start > h->file_size) { set_error("wpk data_start %llu exceeds file size %llu", (unsigned long long)hd.data_start, (unsigned long long)h->file_size); return fail(MC_E_MODEL_MISMATCH); }
    if (hd.toc_offset + (uint64_t)hd.section_count * sizeof(WpkToc) > hd.data_start) {
        set_error("wpk TOC of %u sections runs past data_start=%llu", hd.section_count, (unsigned long long)hd.data_start);
        return fail(MC_E_MODEL_MISMATCH);
    }
    h->toc.resize(hd.section_count);
    if (hd.section_count > 0 && (std::fseek(f, (long)hd.toc_offset, SEEK_SET) != 0 ||
                                 std::fread(h->toc.data(), sizeof(WpkToc), hd.section_count, f) != hd.section_count)) {
        set_error("wpk read TOC failed (%u sections)", hd.section_count);
        return fail(MC_E_IO);
    }
    for (size_t i = 0; i < h->toc.size(); ++i) {
        const WpkToc& t = h->toc[i];
        for (size_t j = 0; j < i; ++j)
            if (h->toc[j].name_hash == t.name_hash) {
                set_error("wpk TOC has duplicate name_hash 0x%016llx", (unsigned long long)t.name_hash);
                return fail(MC_E_MODEL_MISMATCH);
            }
        if ((t.dtype != 0 && t.dtype != 2) || t.layout != 0 || t.rank == 0 || t.rank > 8) {
            set_error("wpk section %zu: unsupported dtype=%u layout=%u rank=%u", i, t.dtype, t.layout, t.rank);
            return fail(MC_E_MODEL_MISMATCH);
        }
        uint64_t elems = 1;
        for (uint32_t r = 0; r < t.rank; ++r) elems *= t.dims[r];
        const uint64_t want = elems * (t.dtype == 0 ? 2u : 1u);
        if (t.data_bytes != want || (t.data_offset & 255u) != 0 || t.data_offset < hd.data_start ||
            t.data_offset + t.data_bytes > h->file_size) {
            set_error("wpk section %zu: data range [%llu,+%llu) invalid (want %llu bytes, 256-byte aligned, inside the file)", i,
                      (unsigned long long)t.data_offset, (unsigned long long)t.data_bytes, (unsigned long long)want);
            return fail(MC_E_MODEL_MISMATCH);
        }
        if (t.dtype == 2) {
            if (t.scale_bytes != (uint64_t)t.dims[0] * 4u || t.scale_offset + t.scale_bytes > h->file_size || t.scale_offset < hd.data_start) {
                set_error("wpk section %zu: scale range invalid", i);
                return fail(MC_E_MODEL_MISMATCH);
            }
        } else if (t.scale_bytes != 0 || t.scale_offset != 0) {
            set_error("wpk section %zu: bf16 section carries scales", i);
            return fail(MC_E_MODEL_MISMATCH);
        }
    }
    *out = h;
    return MC_OK;
}

void mc_sm100_wpk_close(mc_sm100_wpk_t h) {
    if (h == nullptr) return;
    if (h->f) std::fclose(h->f);
    delete h;
}

uint32_t mc_sm100_wpk_section_count(mc_sm100_wpk_t h) { return h ? (uint32_t)h->toc.size() : 0u; }

mc_status_t mc_sm100_wpk_find(mc_sm100_wpk_t h, const char* name, mc_sm100_wpk_section_t* out) {
    clear_error();
    if (h == nullptr || name == nullptr || out == nullptr) { set_error("mc_sm100_wpk_find: invalid args"); return MC_E_INVALID_ARGUMENT; }
    const WpkToc* t = find_section(h, name);
    if (t == nullptr) { set_error("wpk missing section '%s' (fnv1a=0x%016llx)", name, (unsigned long long)fnv1a64(name)); return MC_E_MODEL_MISMATCH; }
    out->name_hash = t->name_hash; out->dtype = t->dtype; out->layout = t->layout; out->rank = t->rank;
    std::memcpy(out->dims, t->dims, sizeof(out->dims));
    out->data_offset = t->data_offset; out->data_bytes = t->data_bytes;
    out->scale_offset = t->scale_offset; out->scale_bytes = t->scale_bytes;
    return MC_OK;
}

// Rows [row_lo, row_hi) of a section into device memory.  interleave != 0: the section is a fused
// gate|up tensor [2*I, K]; the range counts (gate_j, up_j) PAIRS of I and the destination receives
// rows gate[lo], up[lo], gate[lo+1], ... (scales likewise).  Pageable staging, 32 MiB at a time;
// the call returns after the last copy has completed (a load-time call, not a step-time one).
mc_status_t mc_sm100_wpk_upload(mc_sm100_wpk_t h, const char* name, uint32_t row_lo, uint32_t row_hi, int32_t interleave,
                                void* d_data, uint64_t data_capacity, float* d_scale, void* stream) {
    clear_error();
    if (h == nullptr || name == nullptr || d_data == nullptr || row_hi < row_lo) { set_error("mc_sm100_wpk_upload: invalid args"); return MC_E_INVALID_ARGUMENT; }
    const WpkToc* t = find_section(h, name);
    if (t == nullptr) { set_error("wpk missing section '%s'", name); return MC_E_MODEL_MISMATCH; }
    const uint64_t rows = t->dims[0];
    uint64_t row_bytes = t->dtype == 0 ? 2u : 1u;
    for (uint32_t r = 1; r < t->rank; ++r) row_bytes *= t->dims[r];
    const uint64_t limit = interleave ? rows / 2 : rows;
    if ((interleave && (rows & 1u)) || row_hi > limit) { set_error("wpk upload '%s': rows [%u,%u) outside %llu", name, row_lo, row_hi, (unsigned long long)limit); return MC_E_INVALID_ARGUMENT; }
    const uint64_t out_rows = (uint64_t)(row_hi - row_lo) * (interleave ? 2u : 1u);
    if (out_rows * row_bytes > data_capacity) { set_error("wpk upload '%s': needs %llu bytes, destination holds %llu", name, (unsigned long long)(out_rows * row_bytes), (unsigned long long)data_capacity); return MC_E_INVALID_ARGUMENT; }
    if (t->dtype == 2 && d_scale == nullptr) { set_error("wpk upload '%s': e4m3 section needs a scale destination", name); return MC_E_INVALID_ARGUMENT; }
    const cudaStream_t st = (cudaStream_t)stream;
    const uint64_t chunk_rows = std::max<uint64_t>(2, ((32ull << 20) / row_bytes) & ~1ull);
    std::vector<uint8_t> stage((size_t)std::min<uint64_t>(chunk_rows, std::max<uint64_t>(out_rows, 1)) * row_bytes);
    auto read_rows = [&](uint64_t file_off, uint64_t first, uint64_t count, uint64_t elem, uint8_t* dst, uint64_t dst_stride) -> bool {
        // `count` rows of `elem` bytes starting at row `first`, written `dst_stride` apart
        if (dst_stride == elem) {
            return std::fseek(h->f, (long)(file_off + first * elem), SEEK_SET) == 0 && std::fread(dst, elem, count, h->f) == count;
        }
        for (uint64_t r = 0; r < count; ++r)
            if (std::fseek(h->f, (long)(file_off + (first + r) * elem), SEEK_SET) != 0 || std::fread(dst + r * dst_stride, elem, 1, h->f) != 1) return false;
        return true;
    };
    auto push = [&](uint64_t file_off, uint64_t elem, uint8_t* d_dst) -> mc_status_t {
        // uploads the selected rows of an array of `rows` records of `elem` bytes
        const uint64_t per = std::max<uint64_t>(2, (stage.size() / elem) & ~1ull);
        for (uint64_t done = 0; done < out_rows; done += per) {
            const uint64_t n = std::min(per, out_rows - done);
            bool ok;
            if (!interleave) {
                ok = read_rows(file_off, row_lo + done, n, elem, stage.data(), elem);
            } else {
                const uint64_t p0 = row_lo + done / 2, np = n / 2;     // n is even: pairs
                ok = read_rows(file_off, p0, np, elem, stage.data(), 2 * elem) &&
                     read_rows(file_off, rows / 2 + p0, np, elem, stage.data() + elem, 2 * elem);
            }
            if (!ok) { set_error("wpk upload '%s': short read", name); return MC_E_IO; }
            cudaError_t e = cudaMemcpyAsync(d_dst + done * elem, stage.data(), n * elem, cudaMemcpyHostToDevice, st);
            if (e == cudaSuccess) e = cudaStreamSynchronize(st);
            if (e != cudaSuccess) { set_error("wpk upload '%s': copy failed: %s", name, cudaGetErrorString(e)); return MC_E_CUDA; }
        }
        return MC_OK;
    };
    if (stage.size() < 8) stage.resize(8);
    mc_status_t rc = push(t->data_offset, row_bytes, (uint8_t*)d_data);
    if (rc == MC_OK && t->dtype == 2) rc = push(t->scale_offset, 4, (uint8_t*)d_scale);
    return rc;
}

// ---- writer + quantiser (role of tools/quantize.py and the writer of tools/minicpm_common.py) ----

mc_status_t mc_sm100_quantize_rows_host(const uint16_t* h_w, uint32_t N, uint32_t K, uint8_t* h_q, float* h_scale) {
    clear_error();
    if (h_w == nullptr || h_q == nullptr || h_scale == nullptr || N == 0 || K == 0) {
        set_error("mc_sm100_quantize_rows_host: invalid args (N=%u K=%u)", N, K);
        return MC_E_INVALID_ARGUMENT;
    }
    for (uint32_t n = 0; n < N; ++n) {
        const uint16_t* row = h_w + (size_t)n * K;
        float amax = 0.f;
        for (uint32_t k = 0; k < K; ++k) {
            const float a = std::fabs(bf16_bits_to_f32(row[k]));
            if (a > amax || a != a) amax = a != a ? amax : a;
        }
        float sc = amax / 448.0f;                       // fp32 division, floored (minicpm_common.py:204-207)
        if (!(sc > 1e-12f)) sc = 1e-12f;
        h_scale[n] = sc;
        for (uint32_t k = 0; k < K; ++k) h_q[(size_t)n * K + k] = e4m3_from_f32(bf16_bits_to_f32(row[k]) / sc);
    }
    return MC_OK;
}

mc_status_t mc_sm100_e4m3_from_f32_host(const float* h_in, uint64_t n, uint8_t* h_out) {
    clear_error();
    if ((h_in == nullptr || h_out == nullptr) && n != 0) { set_error("mc_sm100_e4m3_from_f32_host: invalid args"); return MC_E_INVALID_ARGUMENT; }
    for (uint64_t i = 0; i < n; ++i) h_out[i] = e4m3_from_f32(h_in[i]);
    return MC_OK;
}

mc_status_t mc_sm100_wpk_writer_create(const char* path, uint32_t max_sections, uint32_t target_sm, const uint8_t* model_hash32,
                                       mc_sm100_wpk_writer_t* out) {
    clear_error();
    if (out != nullptr) *out = nullptr;
    if (path == nullptr || out == nullptr || max_sections == 0 || (target_sm != 100u && target_sm != 120u)) {
        set_error("mc_sm100_wpk_writer_create: invalid args (max_sections=%u target_sm=%u)", max_sections, target_sm);
        return MC_E_INVALID_ARGUMENT;
    }
    FILE* f = std::fopen(path, "wb");
    if (f == nullptr) { set_error("wpk: cannot create '%s'", path); return MC_E_IO; }
    mc_sm100_wpk_writer* w = new (std::nothrow) mc_sm100_wpk_writer();
    if (w == nullptr) { std::fclose(f); set_error("wpk: out of host memory"); return MC_E_OUT_OF_MEMORY; }
    w->f = f;
    w->path = path;
    std::memset(&w->hdr, 0, sizeof(w->hdr));
    w->hdr.magic = 0x31504B4Du;
    w->hdr.abi_version = 2;
    w->hdr.target_sm = (uint16_t)target_sm;
    if (model_hash32 != nullptr) std::memcpy(w->hdr.model_hash, model_hash32, 32);
    w->hdr.toc_offset = 64;
    w->hdr.data_start = (64u + (uint64_t)max_sections * sizeof(WpkToc) + 255u) & ~(uint64_t)255u;
    w->max_sections = max_sections;
    w->cursor = w->hdr.data_start;
    *out = w;
    return MC_OK;
}

mc_status_t mc_sm100_wpk_writer_add(mc_sm100_wpk_writer_t w, const char* name, uint32_t dtype, uint32_t rank, const uint32_t* dims,
                                    const void* h_data, const float* h_scales) {
    clear_error();
    if (w == nullptr || name == nullptr || dims == nullptr || h_data == nullptr || rank == 0 || rank > 8 || (dtype != 0 && dtype != 2) ||
        (dtype == 2) != (h_scales != nullptr)) {
        set_error("mc_sm100_wpk_writer_add: invalid args (dtype=%u rank=%u)", dtype, rank);
        return MC_E_INVALID_ARGUMENT;
    }
    if (w->toc.size() >= w->max_sections) { set_error("wpk writer: more than the %u sections announced", w->max_sections); return MC_E_INVALID_ARGUMENT; }
    WpkToc t;
    std::memset(&t, 0, sizeof(t));
    t.name_hash = fnv1a64(name);
    for (const auto& o : w->toc)
        if (o.name_hash == t.name_hash) { set_error("wpk writer: section '%s' twice", name); return MC_E_INVALID_ARGUMENT; }
    t.dtype = dtype; t.layout = 0; t.rank = rank;
    uint64_t elems = 1;
    for (uint32_t r = 0; r < rank; ++r) { t.dims[r] = dims[r]; elems *= dims[r]; }
    t.data_offset = w->cursor;
    t.data_bytes = elems * (dtype == 0 ? 2u : 1u);
    bool ok = std::fseek(w->f, (long)t.data_offset, SEEK_SET) == 0 && (t.data_bytes == 0 || std::fwrite(h_data, 1, t.data_bytes, w->f) == t.data_bytes);
    uint64_t end = t.data_offset + t.data_bytes;
    if (dtype == 2) {                 // fp32 row scales directly behind the codes (tools/quantize.py:85-113)
        t.scale_offset = end;
        t.scale_bytes = (uint64_t)dims[0] * 4u;
        ok = ok && std::fwrite(h_scales, 1, t.scale_bytes, w->f) == t.scale_bytes;
        end += t.scale_bytes;
    }
    if (!ok) { set_error("wpk writer: write of section '%s' failed", name); return MC_E_IO; }
    w->cursor = (end + 255u) & ~(uint64_t)255u;
    w->toc.push_back(t);
    return MC_OK;
}

mc_status_t mc_sm100_wpk_writer_finish(mc_sm100_wpk_writer_t w) {
    clear_error();
    if (w == nullptr) { set_error("mc_sm100_wpk_writer_finish: invalid args"); return MC_E_INVALID_ARGUMENT; }
    w->hdr.section_count = (uint32_t)w->toc.size();
    bool ok = std::fseek(w->f, 0, SEEK_SET) == 0 && std::fwrite(&w->hdr, sizeof(WpkHeader), 1, w->f) == 1 &&
              (w->toc.empty() || std::fwrite(w->toc.data(), sizeof(WpkToc), w->toc.size(), w->f) == w->toc.size());
    // pad the file to the aligned end, as the packer does
    if (ok && w->cursor > 0) {
        ok = std::fseek(w->f, 0, SEEK_END) == 0;
        const uint64_t have = ok ? (uint64_t)std::ftell(w->f) : 0;
        if (ok && have < w->cursor) {
            const std::vector<uint8_t> zeros((size_t)(w->cursor - have), 0);
            ok = std::fwrite(zeros.data(), 1, zeros.size(), w->f) == zeros.size();
        }
    }
    ok = (std::fclose(w->f) == 0) && ok;
    const std::string path = w->path;
    delete w;
    if (!ok) { set_error("wpk writer: finishing '%s' failed", path.c_str()); return MC_E_IO; }
    return MC_OK;
}

void mc_sm100_wpk_writer_abort(mc_sm100_wpk_writer_t w) {
    if (w == nullptr) return;
    std::fclose(w->f);
    std::remove(w->path.c_str());
    delete w;
}

}  // extern "C"
