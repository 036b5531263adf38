// File IO and quantisation codecs of the host runtime (see io_quant.cpp).
#pragma once

#include <map>
#include <string>
#include <vector>

#include "ps_runtime.h"

namespace psrt {

struct JValue {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    double num = 0;
    std::string str;
    std::vector<JValue> arr;
    std::vector<std::pair<std::string, JValue>> obj;
    const JValue* get(const std::string& key) const;
};
JValue json_parse(const char* data, size_t n);

struct TensorSpec { std::string dtype; std::vector<int64_t> shape; uint64_t begin = 0, end = 0; };
size_t dtype_size(const std::string& dt);

// mmap-backed, zero-copy reader of one .safetensors file
class SafetensorsReader {
public:
    explicit SafetensorsReader(const std::string& path);
    ~SafetensorsReader();
    const std::vector<std::string>& names() const { return names_; }
    const TensorSpec& spec(const std::string& name) const;
    const uint8_t* data(const std::string& name) const;
    const std::map<std::string, std::string>& metadata() const { return metadata_; }
    bool has(const std::string& name) const { return specs_.count(name) != 0; }
    void close();
private:
    std::string path_;
    int fd_ = -1;
    const uint8_t* base_ = nullptr;
    size_t size_ = 0, data_begin_ = 0;
    std::vector<std::string> names_;
    std::map<std::string, TensorSpec> specs_;
    std::map<std::string, std::string> metadata_;
};

// plan -> header -> streamed chunk writes -> fsync
class SafetensorsWriter {
public:
    explicit SafetensorsWriter(const std::string& path);
    ~SafetensorsWriter();
    void set_metadata(const std::string& k, const std::string& v);
    void plan_tensor(const std::string& name, const std::string& dtype, const std::vector<int64_t>& shape);
    void write_header();
    void write_chunk(const std::string& name, const uint8_t* data, size_t n);
    uint32_t tensor_crc(const std::string& name) const;
    void finish();
private:
    struct Planned { TensorSpec spec; uint64_t written = 0; uint32_t crc = 0; };
    std::string path_;
    int fd_ = -1;
    bool header_written_ = false;
    uint64_t cursor_ = 0, data_begin_ = 0;
    std::vector<std::string> order_;
    std::map<std::string, Planned> planned_;
    std::map<std::string, std::string> metadata_;
};

float e4m3_decode(uint8_t b);
uint8_t e4m3_encode(float x);
float e2m1_decode(uint8_t nibble);
uint8_t e2m1_encode(float x);
float ue8m0_decode(uint8_t e);
// One weight row -> canonical NVFP4 (codes k_padded/2 bytes, scales k_padded/16 bytes) / MXFP8 payload.
int kv_nvfp4_row_bytes(int d);
void kv_nvfp4_encode_row(const float* x, int d, uint8_t* row, float* row_scale);
void kv_nvfp4_decode_row(const uint8_t* row, float row_scale, int d, float* out);
void quantize_row_nvfp4(const float* w, int k, int k_padded, float tensor_scale, int search, const float* importance,
                        uint8_t* codes, uint8_t* scales);
void quantize_row_mxfp8(const float* w, int k, int k_padded, int search, const float* importance, uint8_t* codes,
                        uint8_t* scales);

}  // namespace psrt
