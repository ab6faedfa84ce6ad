#include "weights/safetensors.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstdio>
#include <fstream>
#include <functional>
#include <set>
#include <sstream>

namespace illm {

const void* TensorRecord::data() const { return file->data_section() + begin; }

static std::string shape_str(const std::vector<long long>& s) {
    std::string out = "[";
    for (size_t i = 0; i < s.size(); i++) out += (i ? ", " : "") + std::to_string(s[i]);
    return out + "]";
}

SafetensorsFile::SafetensorsFile(const std::string& path) : path_(path) {
    fd_ = ::open(path.c_str(), O_RDONLY);
    if (fd_ < 0) throw WeightError(path + ": cannot be opened");
    struct stat st;
    if (fstat(fd_, &st) != 0) { ::close(fd_); throw WeightError(path + ": cannot be read"); }
    size_ = (size_t)st.st_size;
    auto fail = [&](const std::string& what) {
        if (map_) munmap(map_, size_);
        ::close(fd_);
        fd_ = -1;
        map_ = nullptr;
        throw WeightError(path + ": " + what);
    };
    if (size_ < 8) fail("too short to be a safetensors file");
    map_ = (unsigned char*)mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
    if (map_ == MAP_FAILED) { map_ = nullptr; fail("cannot be mapped into memory"); }
    unsigned long long n = 0;
    for (int i = 7; i >= 0; i--) n = (n << 8) | map_[i];
    if (n > size_ - 8) fail("header length " + std::to_string(n) + " exceeds the file size " + std::to_string(size_));
    Json header;
    try {
        header = Json::parse(std::string((const char*)map_ + 8, (size_t)n));
    } catch (const std::runtime_error& e) {
        fail(std::string("header is not valid JSON (") + e.what() + ")");
    }
    if (!header.is_object()) fail("header is not valid JSON (not an object)");
    base_ = 8 + (size_t)n;
    for (auto& m : header.members()) {
        if (m.first == "__metadata__") { metadata_ = m.second; continue; }
        const Json& rec = m.second;
        TensorRecord r;
        r.name = m.first;
        r.file = this;
        if (!rec.is_object() || !rec.at("dtype").is_string() || !rec.at("shape").is_array() || !rec.at("data_offsets").is_array() ||
            rec.at("data_offsets").size() != 2)
            fail("tensor '" + m.first + "' has a malformed record");
        if (!dtype_from_name(rec.at("dtype").as_string(), &r.dtype))
            fail("tensor '" + m.first + "' has unsupported dtype " + rec.at("dtype").as_string());
        for (const Json& s : rec.at("shape").items()) r.shape.push_back(s.as_int());
        const long long b = rec.at("data_offsets")[0].as_int(), e = rec.at("data_offsets")[1].as_int();
        const long long want = r.numel() * (long long)dtype_size(r.dtype);
        if (e - b != want || b < 0 || base_ + (size_t)e > size_)
            fail("tensor '" + m.first + "' " + shape_str(r.shape) + " " + dtype_name(r.dtype) + " needs " + std::to_string(want) +
                 " bytes, its record gives [" + std::to_string(b) + ", " + std::to_string(e) + ") in a data section of " +
                 std::to_string(size_ - base_) + " bytes (truncated or corrupt file)");
        r.begin = (size_t)b;
        r.end = (size_t)e;
        records_[m.first] = r;
    }
}

SafetensorsFile::~SafetensorsFile() {
    if (map_) munmap(map_, size_);
    if (fd_ >= 0) ::close(fd_);
}

static bool is_file(const std::string& p) {
    struct stat st;
    return stat(p.c_str(), &st) == 0 && S_ISREG(st.st_mode);
}

ModelFiles open_model_files(const std::string& folder) {
    const std::string single = folder + "/model.safetensors", index = folder + "/model.safetensors.index.json";
    ModelFiles out;
    if (is_file(single)) {
        out.files.emplace_back(new SafetensorsFile(single));
    } else if (is_file(index)) {
        std::ifstream f(index);
        std::stringstream ss;
        ss << f.rdbuf();
        Json j;
        try {
            j = Json::parse(ss.str());
        } catch (const std::runtime_error& e) {
            throw WeightError(index + ": not valid JSON (" + e.what() + ")");
        }
        std::set<std::string> shards;
        if (j.at("weight_map").is_object())
            for (auto& m : j.at("weight_map").members())
                if (m.second.is_string()) shards.insert(m.second.as_string());
        for (const std::string& shard : shards) {
            const std::string p = folder + "/" + shard;
            if (!is_file(p)) throw WeightError(index + " names shard '" + shard + "', which is not in " + folder);
            out.files.emplace_back(new SafetensorsFile(p));
        }
    } else {
        throw WeightError(folder + ": neither model.safetensors nor model.safetensors.index.json found");
    }
    for (auto& f : out.files)
        for (auto& r : f->records()) {
            auto it = out.records.find(r.first);
            if (it != out.records.end())
                throw WeightError("tensor '" + r.first + "' appears in both " + it->second.file->path() + " and " + f->path());
            out.records[r.first] = r.second;
        }
    return out;
}

void write_safetensors(const std::string& path, const std::vector<TensorToWrite>& tensors,
                       const std::function<void(size_t, void*, size_t)>& fill, const Json& metadata) {
    Json header = Json::object();
    if (metadata.is_object() && metadata.size()) {
        Json md = Json::object();
        for (auto& m : metadata.members()) md.set(m.first, m.second.is_string() ? m.second : Json(m.second.dump()));
        header.set("__metadata__", md);
    }
    size_t off = 0, largest = 0;
    for (const TensorToWrite& t : tensors) {
        long long n = 1;
        for (long long s : t.shape) n *= s;
        const size_t bytes = (size_t)n * dtype_size(t.dtype);
        Json rec = Json::object(), shape = Json::array(), offs = Json::array();
        for (long long s : t.shape) shape.push(s);
        offs.push((long long)off);
        offs.push((long long)(off + bytes));
        rec.set("dtype", dtype_name(t.dtype));
        rec.set("shape", shape);
        rec.set("data_offsets", offs);
        header.set(t.name, rec);
        off += bytes;
        largest = std::max(largest, bytes);
    }
    std::string blob = header.dump();
    blob.append((8 - blob.size() % 8) % 8, ' ');
    FILE* f = fopen(path.c_str(), "wb");
    if (!f) throw WeightError(path + ": cannot be written");
    unsigned char len[8];
    unsigned long long n = blob.size();
    for (int i = 0; i < 8; i++) len[i] = (unsigned char)(n >> (8 * i));
    std::vector<unsigned char> buf(largest);
    bool ok = fwrite(len, 1, 8, f) == 8 && fwrite(blob.data(), 1, blob.size(), f) == blob.size();
    for (size_t i = 0; ok && i < tensors.size(); i++) {
        long long cnt = 1;
        for (long long s : tensors[i].shape) cnt *= s;
        const size_t bytes = (size_t)cnt * dtype_size(tensors[i].dtype);
        if (!bytes) continue;
        fill(i, buf.data(), bytes);
        ok = fwrite(buf.data(), 1, bytes, f) == bytes;
    }
    ok = (fclose(f) == 0) && ok;
    if (!ok) throw WeightError(path + ": writing failed (disk full?)");
}

}  // namespace illm
