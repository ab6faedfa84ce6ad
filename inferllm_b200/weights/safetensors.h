// Reading and writing the safetensors container (one file, or shards with an index).
//
// Layout of a file: an unsigned 64-bit little-endian header length, a JSON header
// {name: {"dtype", "shape", "data_offsets": [begin, end]}} (offsets relative to the end of the
// header), then the raw little-endian row-major data.  The reference has its own container with the
// same idea, a per-tensor record of dims, name and type followed by the raw data
// (src/core/graph.cpp:285-309); there the bytes are read at first use (optionally through mmap,
// src/file.cpp:15-20), here a file is always memory-mapped and each tensor is copied to the device
// once at load.
#pragma once
#include <functional>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "util/dtype.h"
#include "util/error.h"
#include "util/json.h"

namespace illm {

class SafetensorsFile;

struct TensorRecord {
    std::string name;
    DType dtype = DType::F32;
    std::vector<long long> shape;
    size_t begin = 0, end = 0;             // within the file's data section
    const SafetensorsFile* file = nullptr;
    long long numel() const { long long n = 1; for (long long s : shape) n *= s; return n; }
    const void* data() const;              // the mapped bytes (valid while the file is open)
};

// A memory-mapped safetensors file.  Every record is checked against the file's size when the file
// is opened: a truncated or corrupt file is a WeightError here, not a fault later.
class SafetensorsFile {
public:
    explicit SafetensorsFile(const std::string& path);
    ~SafetensorsFile();
    SafetensorsFile(const SafetensorsFile&) = delete;
    const std::string& path() const { return path_; }
    const std::map<std::string, TensorRecord>& records() const { return records_; }
    const Json& metadata() const { return metadata_; }
    const unsigned char* data_section() const { return map_ + base_; }

private:
    std::string path_;
    int fd_ = -1;
    unsigned char* map_ = nullptr;
    size_t size_ = 0, base_ = 0;
    std::map<std::string, TensorRecord> records_;
    Json metadata_;
};

struct ModelFiles {
    std::vector<std::unique_ptr<SafetensorsFile>> files;
    std::map<std::string, TensorRecord> records;       // all tensors of the folder by name
};
// All tensor records of a model folder: model.safetensors, or the shards named by
// model.safetensors.index.json.
ModelFiles open_model_files(const std::string& folder);

// Writing: the header needs every shape before the data, so the tensors are described first and
// their bytes are produced one tensor at a time by `fill(index, destination)`.
struct TensorToWrite {
    std::string name;
    DType dtype;
    std::vector<long long> shape;
};
void write_safetensors(const std::string& path, const std::vector<TensorToWrite>& tensors,
                       const std::function<void(size_t index, void* dst, size_t bytes)>& fill, const Json& metadata = Json());

}  // namespace illm
