// GGUF container reader and device-resident layer streamer (include/gguf_loader.h).
#include "../../include/gguf_loader.h"

#include <cuda_runtime.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>

namespace b200_llm {

// Forward-only reader over the mapped bytes; every take_* checks the remaining length first and latches `ok` to false
// on the first short read, so a parser can run a whole record and test once.
struct GgufFile::Cursor {
    const uint8_t* p;
    size_t n, at = 0;
    bool ok = true;
    bool need(size_t k) { if (!ok || k > n - at) { ok = false; return false; } return true; }
    uint8_t take8() { if (!need(1)) return 0; return p[at++]; }
    uint16_t take16() { if (!need(2)) return 0; uint16_t v = le16(p + at); at += 2; return v; }
    uint32_t take32() { if (!need(4)) return 0; uint32_t v = le32(p + at); at += 4; return v; }
    uint64_t take64() { if (!need(8)) return 0; uint64_t v = le64(p + at); at += 8; return v; }
    std::string take_string() {
        const uint64_t len = take64();
        if (!ok || len > n - at) { ok = false; return std::string(); }
        std::string s(reinterpret_cast<const char*>(p + at), (size_t)len);
        at += (size_t)len;
        return s;
    }
    bool take_value(GgufType t, GgufValue& v, int depth) {
        v.type = t;
        switch (t) {
            case GgufType::U8: v.u = take8(); break;
            case GgufType::I8: v.i = (int8_t)take8(); break;
            case GgufType::U16: v.u = take16(); break;
            case GgufType::I16: v.i = (int16_t)take16(); break;
            case GgufType::U32: v.u = take32(); break;
            case GgufType::I32: v.i = (int32_t)take32(); break;
            case GgufType::U64: v.u = take64(); break;
            case GgufType::I64: v.i = (int64_t)take64(); break;
            case GgufType::BOOL: v.u = take8() ? 1 : 0; break;
            case GgufType::F32: { const uint32_t b = take32(); float f; std::memcpy(&f, &b, 4); v.f = f; break; }
            case GgufType::F64: { const uint64_t b = take64(); double d; std::memcpy(&d, &b, 8); v.f = d; break; }
            case GgufType::STRING: v.s = take_string(); break;
            case GgufType::ARRAY: {
                const GgufType item = (GgufType)take32();
                const uint64_t count = take64();
                // every item takes at least one byte: a count beyond the bytes that are left is a corrupt file,
                // not a reason to reserve memory for it
                if (!ok || depth > 4 || count > n - at) { ok = false; return false; }
                v.items.resize((size_t)count);
                for (uint64_t k = 0; k < count && ok; k++) take_value(item, v.items[(size_t)k], depth + 1);
                break;
            }
            default: ok = false;
        }
        return ok;
    }
};

bool GgufFile::fail(const std::string& why) { error_ = why; return false; }

void GgufFile::close() {
    if (mapped_ && base_) munmap(const_cast<uint8_t*>(base_), size_);
    base_ = nullptr; size_ = 0; mapped_ = false;
    version_ = 0; alignment_ = 32; data_offset_ = 0;
    meta_.clear(); tensors_.clear(); by_name_.clear();
}

bool GgufFile::open(const std::string& path) {
    close();
    const int fd = ::open(path.c_str(), O_RDONLY);
    if (fd < 0) return fail("cannot open " + path);
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 24) { ::close(fd); return fail("file shorter than a GGUF header: " + path); }
    void* m = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);                                   // the mapping keeps the file alive
    if (m == MAP_FAILED) return fail("mmap failed: " + path);
    base_ = static_cast<const uint8_t*>(m); size_ = (size_t)st.st_size; mapped_ = true;
    if (!parse_all()) { const std::string e = error_; close(); error_ = e; return false; }
    return true;
}

bool GgufFile::parse(const uint8_t* data, size_t size) {
    close();
    if (!data || size < 24) return fail("buffer shorter than a GGUF header");
    base_ = data; size_ = size; mapped_ = false;
    if (!parse_all()) { const std::string e = error_; close(); error_ = e; return false; }
    return true;
}

uint64_t GgufFile::payload_bytes(uint32_t type, uint64_t elements) {
    switch (type) {
        case GGML_F32: return elements * 4;
        case GGML_F16: return elements * 2;
        case GGML_Q4_0: return elements % 32 ? 0 : elements / 32 * 18;
        case GGML_Q8_0: return elements % 32 ? 0 : elements / 32 * 34;
        case GGML_PRISM_Q2_0: return elements % 128 ? 0 : elements / 128 * 34;
        default: return 0;
    }
}

QuantFormat GgufFile::format_of(uint32_t type) {
    switch (type) {
        case GGML_Q4_0: return QUANT_Q4_0;
        case GGML_Q8_0: return QUANT_Q8_0;
        case GGML_PRISM_Q2_0: return QUANT_PRISM_Q2_0;
        default: return QUANT_CUSTOM;
    }
}

bool GgufFile::parse_all() {
    Cursor c{base_, size_};
    if (std::memcmp(base_, "GGUF", 4) != 0) return fail("not a GGUF file (magic)");
    c.at = 4;
    version_ = c.take32();
    if (version_ != 2 && version_ != 3) return fail("unsupported GGUF version " + std::to_string(version_));
    const uint64_t n_tensors = c.take64(), n_meta = c.take64();
    if (n_tensors > size_ || n_meta > size_) return fail("implausible table sizes");      // each entry takes more than one byte
    for (uint64_t k = 0; k < n_meta; k++) {
        const std::string key = c.take_string();
        const GgufType t = (GgufType)c.take32();
        GgufValue v;
        if (!c.take_value(t, v, 0)) return fail("truncated or malformed metadata entry " + std::to_string(k) + " (" + key + ")");
        if (key == "general.alignment") {
            alignment_ = (uint32_t)v.u;
            if (alignment_ == 0) alignment_ = 32;
        }
        meta_[key] = std::move(v);
    }
    tensors_.reserve((size_t)n_tensors);
    for (uint64_t k = 0; k < n_tensors; k++) {
        GgufTensor t;
        t.name = c.take_string();
        const uint32_t nd = c.take32();
        if (!c.ok || nd > 8) return fail("truncated or malformed tensor entry " + std::to_string(k));
        for (uint32_t d = 0; d < nd; d++) t.dims.push_back(c.take64());
        t.type = c.take32();
        t.offset = c.take64();
        if (!c.ok) return fail("truncated tensor entry " + std::to_string(k) + " (" + t.name + ")");
        by_name_[t.name] = tensors_.size();
        tensors_.push_back(std::move(t));
    }
    data_offset_ = ((uint64_t)c.at + alignment_ - 1) / alignment_ * alignment_;
    if (!tensors_.empty() && data_offset_ > size_) return fail("file ends before the tensor data");
    // payload sizes: from the type where this library knows it, else the gap to the next payload (or the end of the file)
    std::vector<uint64_t> starts;
    for (const GgufTensor& t : tensors_) starts.push_back(t.offset);
    std::sort(starts.begin(), starts.end());
    for (GgufTensor& t : tensors_) {
        t.bytes = payload_bytes(t.type, t.elements());
        if (t.bytes == 0) {
            auto nx = std::upper_bound(starts.begin(), starts.end(), t.offset);
            const uint64_t end = nx == starts.end() ? (size_ > data_offset_ ? size_ - data_offset_ : 0) : *nx;
            t.bytes = end > t.offset ? end - t.offset : 0;
        }
    }
    return true;
}

const GgufValue* GgufFile::find(const std::string& key) const {
    auto it = meta_.find(key);
    return it == meta_.end() ? nullptr : &it->second;
}
std::string GgufFile::get_string(const std::string& key, const std::string& fallback) const {
    const GgufValue* v = find(key);
    return v && v->type == GgufType::STRING ? v->s : fallback;
}
uint64_t GgufFile::get_uint(const std::string& key, uint64_t fallback) const {
    const GgufValue* v = find(key);
    if (!v) return fallback;
    switch (v->type) {
        case GgufType::U8: case GgufType::U16: case GgufType::U32: case GgufType::U64: case GgufType::BOOL: return v->u;
        default: return fallback;
    }
}
const GgufTensor* GgufFile::tensor(const std::string& name) const {
    auto it = by_name_.find(name);
    return it == by_name_.end() ? nullptr : &tensors_[it->second];
}
const uint8_t* GgufFile::data(const GgufTensor& t) const {
    if (!base_) return nullptr;
    const uint64_t at = data_offset_ + t.offset;
    if (at >= size_ || t.bytes > size_ - at) return nullptr;
    return base_ + at;
}

bool GgufFile::extract_prism_q2_0(const std::string& name, std::vector<block_prism_q2_0>& blocks, uint64_t* K, uint64_t* N) const {
    const GgufTensor* t = tensor(name);
    if (!t || t->dims.empty()) return false;
    const uint64_t n = t->elements();
    if (n == 0 || n % 128 != 0) return false;
    const uint64_t nb = n / 128, at = data_offset_ + t->offset;
    if (at > size_ || nb * 34 > size_ - at) return false;
    blocks.resize((size_t)nb);
    const uint8_t* src = base_ + at;
    for (uint64_t b = 0; b < nb; b++, src += 34) {
        const uint16_t d = le16(src);
        std::memcpy(&blocks[(size_t)b].d, &d, 2);
        std::memcpy(blocks[(size_t)b].qs, src + 2, 32);
    }
    if (K) *K = t->dims[0];
    if (N) *N = t->dims.size() > 1 ? t->dims[1] : 1;
    return true;
}

// ---------------------------------------------------------------------------------------------
// layer streamer
// ---------------------------------------------------------------------------------------------
int GgufLayerStreamer::parse_layer_index(const std::string& name) {
    for (const char* prefix : {"model.layers.", "blk."}) {
        const size_t pl = std::strlen(prefix);
        if (name.compare(0, pl, prefix) != 0) continue;
        size_t i = pl;
        long v = 0;
        while (i < name.size() && name[i] >= '0' && name[i] <= '9' && v < 100000000) { v = v * 10 + (name[i] - '0'); i++; }
        if (i == pl || i >= name.size() || name[i] != '.') return -1;
        return (int)v;
    }
    return -1;
}

bool GgufLayerStreamer::open(const std::string& path, size_t resident_layers, bool upload) {
    close();
    return file_.open(path) && finish_open(resident_layers, upload);
}
bool GgufLayerStreamer::open(const uint8_t* data, size_t size, size_t resident_layers, bool upload) {
    close();
    return file_.parse(data, size) && finish_open(resident_layers, upload);
}

bool GgufLayerStreamer::finish_open(size_t resident_layers, bool upload) {
    budget_ = resident_layers < 1 ? 1 : resident_layers;
    upload_ = upload;
    const auto& ts = file_.tensors();
    for (size_t i = 0; i < ts.size(); i++) {
        if (!file_.data(ts[i])) { close(); return false; }                 // a tensor that leaves the file cannot be served
        Group& g = groups_[parse_layer_index(ts[i].name)];
        g.offsets.push_back(g.bytes);
        g.tensors.push_back(i);
        g.bytes += (ts[i].bytes + 255) / 256 * 256;                        // 256-byte aligned inside the layer's device block
        total_bytes_ += ts[i].bytes;
    }
    auto sh = groups_.find(-1);
    if (sh != groups_.end()) {
        shared_bytes_ = 0;
        for (size_t i : sh->second.tensors) shared_bytes_ += ts[i].bytes;
        if (!make_resident(sh->second)) { close(); return false; }
    }
    if (upload_) {
        cudaStream_t s = nullptr;
        if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) { cudaGetLastError(); close(); return false; }
        copy_stream_ = s;
    }
    return true;
}

void GgufLayerStreamer::close() {
    if (copy_stream_) { cudaStreamSynchronize((cudaStream_t)copy_stream_); cudaStreamDestroy((cudaStream_t)copy_stream_); copy_stream_ = nullptr; }
    for (auto& kv : groups_)
        if (kv.second.device) { cudaFree(kv.second.device); kv.second.device = nullptr; }
    groups_.clear();
    file_.close();
    resident_bytes_ = peak_bytes_ = total_bytes_ = shared_bytes_ = 0;
    tick_ = 0;
}

std::vector<int> GgufLayerStreamer::layer_indices() const {
    std::vector<int> out;
    for (const auto& kv : groups_) if (kv.first >= 0) out.push_back(kv.first);
    return out;
}

std::vector<std::string> GgufLayerStreamer::layer_tensor_names(int layer) const {
    std::vector<std::string> out;
    auto it = groups_.find(layer);
    if (it != groups_.end()) for (size_t i : it->second.tensors) out.push_back(file_.tensors()[i].name);
    return out;
}

bool GgufLayerStreamer::make_resident(Group& g) {
    if (g.resident) return true;
    size_t payload = 0;
    for (size_t i : g.tensors) payload += file_.tensors()[i].bytes;
    if (upload_) {
        if (cudaMalloc(&g.device, g.bytes ? g.bytes : 256) != cudaSuccess) { cudaGetLastError(); g.device = nullptr; return false; }
        cudaStream_t s = (cudaStream_t)copy_stream_;
        for (size_t k = 0; k < g.tensors.size(); k++) {
            const GgufTensor& t = file_.tensors()[g.tensors[k]];
            if (t.bytes == 0) continue;
            if (cudaMemcpyAsync(static_cast<uint8_t*>(g.device) + g.offsets[k], file_.data(t), t.bytes, cudaMemcpyHostToDevice, s) != cudaSuccess) {
                cudaGetLastError(); cudaFree(g.device); g.device = nullptr; return false;
            }
        }
    }
    g.resident = true;
    resident_bytes_ += payload;
    if (resident_bytes_ > peak_bytes_) peak_bytes_ = resident_bytes_;
    return true;
}

// Frees least recently used layers (never `keep`) until at most `allowed` layers are resident.
void GgufLayerStreamer::evict_down_to(size_t allowed, int keep) {
    for (;;) {
        size_t held = 0;
        Group* victim = nullptr;
        for (auto& kv : groups_) {
            if (kv.first < 0 || !kv.second.resident) continue;
            held++;
            if (kv.first == keep) continue;
            if (!victim || kv.second.last_use < victim->last_use) victim = &kv.second;
        }
        if (held <= allowed || !victim) return;
        if (victim->device) {
            if (copy_stream_) cudaStreamSynchronize((cudaStream_t)copy_stream_);
            cudaFree(victim->device);            // waits for kernels that may still read the block
            victim->device = nullptr;
        }
        size_t payload = 0;
        for (size_t i : victim->tensors) payload += file_.tensors()[i].bytes;
        victim->resident = false;
        resident_bytes_ -= payload;
    }
}

bool GgufLayerStreamer::acquire_layer(int layer) {
    auto it = groups_.find(layer);
    if (layer < 0 || it == groups_.end()) return false;
    it->second.last_use = ++tick_;
    if (!make_resident(it->second)) return false;
    evict_down_to(budget_, layer);
    // The layer behind this one is requested now, so that its upload overlaps this layer's compute: with a budget of
    // two or more it takes the slot of the least recently used layer.
    auto nx = std::next(it);
    if (budget_ >= 2 && nx != groups_.end() && !nx->second.resident) {
        evict_down_to(budget_ - 1, layer);
        nx->second.last_use = ++tick_;
        make_resident(nx->second);               // a failed prefetch is not an error: the layer is loaded when it is acquired
    }
    if (copy_stream_) cudaStreamSynchronize((cudaStream_t)copy_stream_);     // this layer's bytes have landed
    return true;
}

bool GgufLayerStreamer::is_resident(int layer) const {
    auto it = groups_.find(layer);
    return it != groups_.end() && it->second.resident;
}

const void* GgufLayerStreamer::tensor_data(const std::string& name) const {
    const GgufTensor* t = file_.tensor(name);
    if (!t) return nullptr;
    auto it = groups_.find(parse_layer_index(name));
    if (it == groups_.end() || !it->second.resident) return nullptr;
    if (!upload_) return file_.data(*t);
    const Group& g = it->second;
    for (size_t k = 0; k < g.tensors.size(); k++)
        if (&file_.tensors()[g.tensors[k]] == t) return static_cast<const uint8_t*>(g.device) + g.offsets[k];
    return nullptr;
}

}  // namespace b200_llm

// ---------------------------------------------------------------------------------------------
// C surface
// ---------------------------------------------------------------------------------------------
using b200_llm::GgufFile;
using b200_llm::GgufLayerStreamer;
using b200_llm::GgufTensor;

namespace {
thread_local std::string t_gguf_error;
int copy_out(const std::string& s, char* out, size_t cap) {
    if (!out || cap == 0) return 0;
    const size_t n = s.size() < cap - 1 ? s.size() : cap - 1;
    std::memcpy(out, s.data(), n);
    out[n] = 0;
    return 1;
}
}  // namespace

extern "C" {

void* b200_gguf_open(const char* path) {
    if (!path) { t_gguf_error = "null path"; return nullptr; }
    GgufFile* f = new GgufFile;
    if (!f->open(path)) { t_gguf_error = f->error(); delete f; return nullptr; }
    return f;
}
void* b200_gguf_parse(const void* data, size_t size) {
    GgufFile* f = new GgufFile;
    if (!f->parse(static_cast<const uint8_t*>(data), size)) { t_gguf_error = f->error(); delete f; return nullptr; }
    return f;
}
void b200_gguf_close(void* file) { delete static_cast<GgufFile*>(file); }
const char* b200_gguf_error(void) { return t_gguf_error.c_str(); }
uint32_t b200_gguf_version(void* f) { return f ? static_cast<GgufFile*>(f)->version() : 0; }
uint32_t b200_gguf_alignment(void* f) { return f ? static_cast<GgufFile*>(f)->alignment() : 0; }
uint64_t b200_gguf_data_offset(void* f) { return f ? static_cast<GgufFile*>(f)->data_offset() : 0; }
uint64_t b200_gguf_tensor_count(void* f) { return f ? static_cast<GgufFile*>(f)->tensor_count() : 0; }
uint64_t b200_gguf_metadata_count(void* f) { return f ? static_cast<GgufFile*>(f)->metadata_count() : 0; }

int b200_gguf_get_uint(void* f, const char* key, uint64_t* value) {
    if (!f || !key || !value) return 0;
    const b200_llm::GgufValue* v = static_cast<GgufFile*>(f)->find(key);
    if (!v) return 0;
    switch (v->type) {
        case b200_llm::GgufType::U8: case b200_llm::GgufType::U16: case b200_llm::GgufType::U32: case b200_llm::GgufType::U64:
        case b200_llm::GgufType::BOOL: *value = v->u; return 1;
        default: return 0;
    }
}
int b200_gguf_get_string(void* f, const char* key, char* out, size_t cap) {
    if (!f || !key) return 0;
    const b200_llm::GgufValue* v = static_cast<GgufFile*>(f)->find(key);
    if (!v || v->type != b200_llm::GgufType::STRING) return 0;
    return copy_out(v->s, out, cap);
}
int b200_gguf_tensor_name(void* f, uint64_t index, char* out, size_t cap) {
    if (!f || index >= static_cast<GgufFile*>(f)->tensor_count()) return 0;
    return copy_out(static_cast<GgufFile*>(f)->tensors()[(size_t)index].name, out, cap);
}
int b200_gguf_tensor_info(void* f, const char* name, uint32_t* n_dims, uint64_t* dims4, uint32_t* type, uint64_t* file_offset, uint64_t* bytes) {
    if (!f || !name) return 0;
    const GgufFile* g = static_cast<GgufFile*>(f);
    const GgufTensor* t = g->tensor(name);
    if (!t) return 0;
    if (n_dims) *n_dims = (uint32_t)t->dims.size();
    if (dims4) for (size_t d = 0; d < 4; d++) dims4[d] = d < t->dims.size() ? t->dims[d] : 1;
    if (type) *type = t->type;
    if (file_offset) *file_offset = g->data_offset() + t->offset;
    if (bytes) *bytes = t->bytes;
    return 1;
}
const void* b200_gguf_tensor_data(void* f, const char* name) { return f && name ? static_cast<GgufFile*>(f)->data(name) : nullptr; }
int b200_gguf_tensor_format(void* f, const char* name) {
    if (!f || !name) return -1;
    const GgufTensor* t = static_cast<GgufFile*>(f)->tensor(name);
    if (!t) return -1;
    const QuantFormat q = GgufFile::format_of(t->type);
    return q == QUANT_CUSTOM ? -1 : (int)q;
}
int64_t b200_gguf_extract_prism_q2_0(void* f, const char* name, void* blocks, uint64_t capacity, uint64_t* K, uint64_t* N) {
    if (!f || !name || !blocks) return -1;
    std::vector<block_prism_q2_0> v;
    if (!static_cast<GgufFile*>(f)->extract_prism_q2_0(name, v, K, N) || v.size() > capacity) return -1;
    std::memcpy(blocks, v.data(), v.size() * sizeof(block_prism_q2_0));
    return (int64_t)v.size();
}

void* b200_gguf_streamer_open(const char* path, uint64_t resident_layers, int upload) {
    if (!path) return nullptr;
    GgufLayerStreamer* s = new GgufLayerStreamer;
    if (!s->open(path, (size_t)resident_layers, upload != 0)) { t_gguf_error = s->file().error(); delete s; return nullptr; }
    return s;
}
void b200_gguf_streamer_close(void* s) { delete static_cast<GgufLayerStreamer*>(s); }
int b200_gguf_streamer_acquire(void* s, int layer) { return s && static_cast<GgufLayerStreamer*>(s)->acquire_layer(layer) ? 1 : 0; }
int b200_gguf_streamer_is_resident(void* s, int layer) { return s && static_cast<GgufLayerStreamer*>(s)->is_resident(layer) ? 1 : 0; }
const void* b200_gguf_streamer_tensor(void* s, const char* name) { return s && name ? static_cast<GgufLayerStreamer*>(s)->tensor_data(name) : nullptr; }
uint64_t b200_gguf_streamer_stat(void* s, int what) {
    if (!s) return 0;
    GgufLayerStreamer* g = static_cast<GgufLayerStreamer*>(s);
    switch (what) {
        case 0: return g->current_resident_bytes();
        case 1: return g->peak_resident_bytes();
        case 2: return g->total_model_bytes();
        case 3: return g->shared_bytes();
        case 4: return g->layer_indices().size();
        default: return 0;
    }
}
int b200_gguf_parse_layer_index(const char* name) { return name ? GgufLayerStreamer::parse_layer_index(name) : -1; }

}  // extern "C"
