// GGUF ingest for the weight formats the projection path decodes.
//
// Role of the reference's GGUFLoader / GGUFLayerStreamer (core/weights/gguf_loader.h:46-127,
// core/weights/gguf_layer_streamer.h:36-95): parse a GGUF v2/v3 container (from a memory-mapped file or from a caller's
// buffer), answer metadata and tensor-directory queries, hand out zero-copy pointers to tensor payloads, and pull a
// PrismML Q2_0 tensor out as block_prism_q2_0 records; on top of it, serve a model layer by layer with a bounded
// number of layers resident.  On a B200 "resident" means resident in HBM: the streamer uploads a layer's tensors to
// the device when the layer is acquired (and the next one behind it) and frees the least recently used layer when
// more than `resident_layers` are held.
//
// Everything is bounds-checked against the buffer: a truncated or corrupt file makes open()/parse() return false, never
// a read outside the mapping.  Multi-byte fields are read byte by byte as little-endian, so the host's byte order does
// not matter.
#pragma once
#ifdef __cplusplus
#include <cstddef>
#include <cstdint>
#include <map>
#include <string>
#include <vector>

#include "quant_router.h"

namespace b200_llm {

enum class GgufType : uint32_t { U8 = 0, I8 = 1, U16 = 2, I16 = 3, U32 = 4, I32 = 5, F32 = 6, BOOL = 7, STRING = 8, ARRAY = 9,
                                 U64 = 10, I64 = 11, F64 = 12 };

struct GgufValue {
    GgufType type = GgufType::U32;
    uint64_t u = 0;                  // unsigned integers and BOOL
    int64_t i = 0;                   // signed integers
    double f = 0.0;                  // F32 / F64
    std::string s;                   // STRING
    std::vector<GgufValue> items;    // ARRAY
};

// ggml tensor type ids of the payloads this library can hand to its kernels unchanged
enum : uint32_t { GGML_F32 = 0, GGML_F16 = 1, GGML_Q4_0 = 2, GGML_Q8_0 = 8, GGML_PRISM_Q2_0 = 100 };

struct GgufTensor {
    std::string name;
    std::vector<uint64_t> dims;      // dims[0] is the contiguous (input, K) dimension, dims[1] the rows (N)
    uint32_t type = 0;               // ggml type id
    uint64_t offset = 0;             // relative to data_offset()
    uint64_t bytes = 0;              // payload size: from the type where it is known, else up to the next tensor / end of file
    uint64_t elements() const { uint64_t n = dims.empty() ? 0 : 1; for (uint64_t d : dims) n *= d; return n; }
};

class GgufFile {
public:
    GgufFile() = default;
    ~GgufFile() { close(); }
    GgufFile(const GgufFile&) = delete;
    GgufFile& operator=(const GgufFile&) = delete;

    bool open(const std::string& path);                       // read-only memory map
    bool parse(const uint8_t* data, size_t size);             // caller keeps `data` alive while this object is open
    void close();

    bool is_open() const { return base_ != nullptr; }
    uint32_t version() const { return version_; }
    uint32_t alignment() const { return alignment_; }
    uint64_t data_offset() const { return data_offset_; }
    size_t file_size() const { return size_; }
    size_t tensor_count() const { return tensors_.size(); }
    size_t metadata_count() const { return meta_.size(); }
    const std::string& error() const { return error_; }

    const GgufValue* find(const std::string& key) const;
    std::string get_string(const std::string& key, const std::string& fallback = "") const;
    uint64_t get_uint(const std::string& key, uint64_t fallback = 0) const;

    const std::vector<GgufTensor>& tensors() const { return tensors_; }          // in file order
    const GgufTensor* tensor(const std::string& name) const;
    // payload of a tensor inside the mapping; nullptr if its declared range leaves the file
    const uint8_t* data(const GgufTensor& t) const;
    const uint8_t* data(const std::string& name) const { const GgufTensor* t = tensor(name); return t ? data(*t) : nullptr; }

    // Payload bytes of `elements` values of ggml type `type`, 0 if the type is not one of the enum above.
    static uint64_t payload_bytes(uint32_t type, uint64_t elements);
    // QuantFormat whose packed layout equals the ggml payload byte for byte (GGML_Q4_0 -> QUANT_Q4_0, GGML_Q8_0 -> QUANT_Q8_0,
    // GGML_PRISM_Q2_0 -> QUANT_PRISM_Q2_0), QUANT_CUSTOM otherwise.
    static QuantFormat format_of(uint32_t type);

    // PrismML Q2_0 tensor as block records (fp16 scale read as little-endian + 32 code bytes); K = dims[0], N = dims[1] (1 if absent).
    // False if the tensor is missing, has no dimensions, its element count is not a multiple of 128, or its blocks leave the file.
    bool extract_prism_q2_0(const std::string& name, std::vector<block_prism_q2_0>& blocks, uint64_t* K = nullptr, uint64_t* N = nullptr) const;

    static uint16_t le16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }
    static uint32_t le32(const uint8_t* p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24); }
    static uint64_t le64(const uint8_t* p) { return (uint64_t)le32(p) | ((uint64_t)le32(p + 4) << 32); }

private:
    struct Cursor;
    bool parse_all();
    bool fail(const std::string& why);

    const uint8_t* base_ = nullptr;
    size_t size_ = 0;
    bool mapped_ = false;
    uint32_t version_ = 0, alignment_ = 32;
    uint64_t data_offset_ = 0;
    std::map<std::string, GgufValue> meta_;
    std::vector<GgufTensor> tensors_;
    std::map<std::string, size_t> by_name_;
    std::string error_;
};

// Layer-by-layer serving with bounded residency in device memory.
class GgufLayerStreamer {
public:
    GgufLayerStreamer() = default;
    ~GgufLayerStreamer() { close(); }
    GgufLayerStreamer(const GgufLayerStreamer&) = delete;
    GgufLayerStreamer& operator=(const GgufLayerStreamer&) = delete;

    // resident_layers >= 1 transformer layers stay on the device at once; tensors outside any layer ("shared":
    // embeddings, final norm, head) are uploaded at open and stay.  upload == false keeps everything on the host
    // (directory and accounting only: usable without a GPU).
    bool open(const std::string& path, size_t resident_layers = 2, bool upload = true);
    bool open(const uint8_t* data, size_t size, size_t resident_layers = 2, bool upload = true);
    void close();
    bool is_open() const { return file_.is_open(); }

    std::vector<int> layer_indices() const;                                   // ascending
    std::vector<std::string> layer_tensor_names(int layer) const;             // layer == -1: the shared group
    // Makes `layer` resident (uploading it if needed), starts the upload of the next layer and frees least recently
    // used layers beyond the budget.  False for an unknown layer or a failed upload.
    bool acquire_layer(int layer);
    bool is_resident(int layer) const;
    // Device pointer of a tensor of a resident layer or of the shared group (host pointer into the mapping when
    // opened with upload == false); nullptr if its layer is not resident.
    const void* tensor_data(const std::string& name) const;

    size_t current_resident_bytes() const { return resident_bytes_; }
    size_t peak_resident_bytes() const { return peak_bytes_; }
    size_t total_model_bytes() const { return total_bytes_; }
    size_t shared_bytes() const { return shared_bytes_; }
    const GgufFile& file() const { return file_; }

    // "model.layers.N.<rest>" or "blk.N.<rest>" -> N; anything else -> -1.
    static int parse_layer_index(const std::string& tensor_name);

private:
    struct Group { std::vector<size_t> tensors; size_t bytes = 0; void* device = nullptr; std::vector<size_t> offsets; uint64_t last_use = 0; bool resident = false; };
    bool finish_open(size_t resident_layers, bool upload);
    bool make_resident(Group& g);
    void evict_down_to(size_t allowed, int keep);

    GgufFile file_;
    std::map<int, Group> groups_;
    size_t budget_ = 2;
    bool upload_ = true;
    uint64_t tick_ = 0;
    size_t resident_bytes_ = 0, peak_bytes_ = 0, total_bytes_ = 0, shared_bytes_ = 0;
    void* copy_stream_ = nullptr;
};

}  // namespace b200_llm

#else   /* C callers see the C entry points below only */
#include <stddef.h>
#include <stdint.h>
#endif

#ifdef __cplusplus
extern "C" {
#endif
/* C surface over GgufFile / GgufLayerStreamer for the Python side (no counterpart in the reference's C ABI: its loader is
 * reached from Objective-C++ only).  Handles are opaque; strings are NUL-terminated UTF-8. */
void* b200_gguf_open(const char* path);
void* b200_gguf_parse(const void* data, size_t size);         /* the caller keeps `data` alive until b200_gguf_close */
void b200_gguf_close(void* file);
const char* b200_gguf_error(void);                             /* why the last open/parse on this thread failed */
uint32_t b200_gguf_version(void* file);
uint32_t b200_gguf_alignment(void* file);
uint64_t b200_gguf_data_offset(void* file);
uint64_t b200_gguf_tensor_count(void* file);
uint64_t b200_gguf_metadata_count(void* file);
/* 1 and the value if the key exists with a compatible type, else 0 */
int b200_gguf_get_uint(void* file, const char* key, uint64_t* value);
int b200_gguf_get_string(void* file, const char* key, char* out, size_t out_bytes);
/* tensor directory: index in file order -> name; name -> dims (up to 4), ggml type, payload offset from the start of the file, bytes */
int b200_gguf_tensor_name(void* file, uint64_t index, char* out, size_t out_bytes);
int b200_gguf_tensor_info(void* file, const char* name, uint32_t* n_dims, uint64_t* dims4, uint32_t* type, uint64_t* file_offset,
                          uint64_t* bytes);
/* host pointer to the payload inside the mapping (NULL if unknown or out of bounds) */
const void* b200_gguf_tensor_data(void* file, const char* name);
/* QuantFormat id whose packed layout equals this tensor's payload, or -1 */
int b200_gguf_tensor_format(void* file, const char* name);
/* Prism Q2_0 extraction into `blocks` (34 bytes each, capacity in blocks); returns the block count or -1 */
int64_t b200_gguf_extract_prism_q2_0(void* file, const char* name, void* blocks, uint64_t capacity_blocks, uint64_t* K, uint64_t* N);

void* b200_gguf_streamer_open(const char* path, uint64_t resident_layers, int upload);
void b200_gguf_streamer_close(void* streamer);
int b200_gguf_streamer_acquire(void* streamer, int layer);
int b200_gguf_streamer_is_resident(void* streamer, int layer);
const void* b200_gguf_streamer_tensor(void* streamer, const char* name);
uint64_t b200_gguf_streamer_stat(void* streamer, int what);   /* 0 current, 1 peak, 2 total, 3 shared bytes, 4 number of layers */
int b200_gguf_parse_layer_index(const char* tensor_name);
#ifdef __cplusplus
}
#endif
