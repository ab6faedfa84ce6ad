#include "weights/loader.h"

#include <sys/stat.h>

#include <algorithm>
#include <cstring>
#include <fstream>

#include "csrc/random_init.h"

namespace illm {

static std::string shape_str(const std::vector<long long>& s) {
    std::string out = "[";
    for (size_t i = 0; i < s.size(); i++) out += (i ? ", " : "") + std::to_string(s[i]);
    return out + "]";
}
static bool ends_with(const std::string& s, const std::string& suffix) {
    return s.size() >= suffix.size() && s.compare(s.size() - suffix.size(), suffix.size(), suffix) == 0;
}

void check_names_and_shapes(const std::vector<std::pair<std::string, TensorDecl>>& decls,
                            const std::map<std::string, TensorRecord>& records) {
    std::map<std::string, const TensorDecl*> by_name;
    for (auto& d : decls) by_name[d.first] = &d.second;
    std::vector<std::string> missing, unexpected, wrong;
    for (auto& d : by_name)
        if (!records.count(d.first)) missing.push_back(d.first);
    for (auto& r : records)
        if (!by_name.count(r.first) && !ends_with(r.first, "rotary_emb.inv_freq")) unexpected.push_back(r.first);
    for (auto& d : by_name) {
        auto it = records.find(d.first);
        if (it != records.end() && it->second.shape != d.second->shape)
            wrong.push_back(d.first + " expected " + shape_str(d.second->shape) + " found " + shape_str(it->second.shape));
    }
    if (missing.empty() && unexpected.empty() && wrong.empty()) return;
    auto join = [](const std::vector<std::string>& v, const char* sep) {
        std::string out;
        for (size_t i = 0; i < v.size(); i++) out += (i ? sep : "") + v[i];
        return out;
    };
    std::string msg = "the weight file does not match the model:";
    if (!missing.empty()) msg += "\n  missing tensors (" + std::to_string(missing.size()) + "): " + join(missing, ", ");
    if (!unexpected.empty()) msg += "\n  unexpected tensors (" + std::to_string(unexpected.size()) + "): " + join(unexpected, ", ");
    if (!wrong.empty()) msg += "\n  wrong shapes (" + std::to_string(wrong.size()) + "): " + join(wrong, "; ");
    throw WeightError(msg);
}

DType storage_dtype(DType stored, DType runtime_dtype, const std::string& init) {
    if (init == "int" || !dtype_is_float(stored)) return DType::I32;
    if (runtime_dtype == DType::F32) return DType::F32;
    if (stored == DType::F32 || stored == DType::F64) return DType::F32;
    return DType::BF16;
}

void check_model_folder(const DecoderModel& model, const std::string& folder) {
    ModelFiles files = open_model_files(folder);
    check_names_and_shapes(model.tensor_decls(), files.records);
}

// ---- sources

namespace {

// Copies `bytes` of host memory to the device through a pinned staging buffer, in pieces.
class Uploader {
public:
    explicit Uploader(Device* dev) : dev_(dev) {
        for (int i = 0; i < 2; i++) stage_[i] = (char*)dev->alloc_pinned(kPiece);
        for (int i = 0; i < 2; i++) check_cuda(cudaEventCreateWithFlags(&done_[i], cudaEventDisableTiming), "cudaEventCreate");
    }
    ~Uploader() {
        dev_->synchronize();
        for (int i = 0; i < 2; i++) {
            dev_->free_pinned(stage_[i]);
            cudaEventDestroy(done_[i]);
        }
    }
    void upload(void* dst, const void* src, size_t bytes) {
        for (size_t off = 0; off < bytes; off += kPiece) {
            const size_t n = std::min(kPiece, bytes - off);
            if (used_[cur_]) check_cuda(cudaEventSynchronize(done_[cur_]), "waiting for an upload");
            memcpy(stage_[cur_], (const char*)src + off, n);
            check_cuda(cudaMemcpyAsync((char*)dst + off, stage_[cur_], n, cudaMemcpyHostToDevice, dev_->stream()), "uploading weights");
            check_cuda(cudaEventRecord(done_[cur_], dev_->stream()), "cudaEventRecord");
            used_[cur_] = true;
            cur_ ^= 1;
        }
    }

private:
    static constexpr size_t kPiece = (size_t)64 << 20;
    Device* dev_;
    char* stage_[2];
    cudaEvent_t done_[2];
    bool used_[2] = {false, false};
    int cur_ = 0;
};

// Puts a contiguous tensor of `have` at `tmp` into `dst` as `want`, rows `dst_row_elems` apart.
void place(Device& dev, const void* tmp, DType have, void* dst, DType want, long long rows, long long cols, long long dst_row_elems) {
    const bool strided = dst_row_elems && dst_row_elems != cols;
    if (!strided) {
        if (have == want) {
            check_cuda(cudaMemcpyAsync(dst, tmp, (size_t)rows * cols * dtype_size(want), cudaMemcpyDeviceToDevice, dev.stream()),
                       "copying a tensor");
        } else {
            ops::convert(dev, tmp, have, dst, want, rows * cols);
        }
        return;
    }
    const void* src = tmp;
    if (have != want) {
        void* conv = dev.alloc((size_t)rows * cols * dtype_size(want));
        ops::convert(dev, tmp, have, conv, want, rows * cols);
        src = conv;
    }
    const size_t es = dtype_size(want);
    check_cuda(cudaMemcpy2DAsync(dst, (size_t)dst_row_elems * es, src, (size_t)cols * es, (size_t)cols * es, (size_t)rows,
                                 cudaMemcpyDeviceToDevice, dev.stream()),
               "interleaving a tensor's rows");
}

void rows_cols(const std::vector<long long>& shape, long long* rows, long long* cols) {
    *cols = shape.empty() ? 1 : shape.back();
    *rows = 1;
    for (size_t i = 0; i + 1 < shape.size(); i++) *rows *= shape[i];
}

class FileSource : public TensorSource {
public:
    FileSource(Runtime* rt, const std::map<std::string, TensorRecord>* records, const std::map<std::string, std::string>* inits,
               std::string prefix, Uploader* up)
            : rt_(rt), records_(records), inits_(inits), prefix_(std::move(prefix)), up_(up) {}
    const TensorRecord& rec(const std::string& name) const { return records_->at(prefix_ + name); }
    DType kept_dtype(const std::string& name) override {
        auto it = inits_->find(prefix_ + name);
        return storage_dtype(rec(name).dtype, rt_->dtype, it == inits_->end() ? "matrix" : it->second);
    }
    std::vector<long long> shape(const std::string& name) override { return rec(name).shape; }
    void fetch_into(const std::string& name, void* dst, DType want, long long dst_row_elems) override {
        const TensorRecord& r = rec(name);
        if (r.numel() == 0) return;
        Device& dev = *rt_->dev;
        dev.arena_rewind();
        void* tmp = dev.alloc((size_t)r.numel() * dtype_size(r.dtype));
        up_->upload(tmp, r.data(), (size_t)r.numel() * dtype_size(r.dtype));
        long long rows, cols;
        rows_cols(r.shape, &rows, &cols);
        place(dev, tmp, r.dtype, dst, want, rows, cols, dst_row_elems);
    }

private:
    Runtime* rt_;
    const std::map<std::string, TensorRecord>* records_;
    const std::map<std::string, std::string>* inits_;
    std::string prefix_;
    Uploader* up_;
};

class RandomSource : public TensorSource {
public:
    RandomSource(Runtime* rt, const std::map<std::string, TensorDecl>* decls, std::string prefix, unsigned long long seed)
            : rt_(rt), decls_(decls), prefix_(std::move(prefix)), seed_(seed) {}
    const TensorDecl& decl(const std::string& name) const { return decls_->at(prefix_ + name); }
    DType kept_dtype(const std::string& name) override {
        if (decl(name).init == "int") return DType::I32;
        return rt_->is_f32() ? DType::F32 : DType::BF16;
    }
    std::vector<long long> shape(const std::string& name) override { return decl(name).shape; }
    void fetch_into(const std::string& name, void* dst, DType want, long long dst_row_elems) override {
        const TensorDecl& d = decl(name);
        if (d.numel() == 0) return;
        Device& dev = *rt_->dev;
        long long rows, cols;
        rows_cols(d.shape, &rows, &cols);
        if (d.init == "int") {
            check_cuda(cudaMemsetAsync(dst, 0, (size_t)d.numel() * 4, dev.stream()), "zeroing an integer table");
            return;
        }
        // generated in the dtype a file of this model would be stored in, then brought to what the part wants
        const DType have = kept_dtype(name);
        dev.arena_rewind();
        void* tmp = dev.alloc((size_t)d.numel() * dtype_size(have));
        ops::fill_random(dev, tmp, have, d.numel(), illm_random_key(seed_, (prefix_ + name).c_str()), 0.02f, d.init == "norm" ? 1.0f : 0.0f);
        place(dev, tmp, have, dst, want, rows, cols, dst_row_elems);
    }

private:
    Runtime* rt_;
    const std::map<std::string, TensorDecl>* decls_;
    std::string prefix_;
    unsigned long long seed_;
};

}  // namespace

void load_model_weights(DecoderModel& model, const std::string& folder) {
    if (!model.rt) throw EngineError("a model without a device cannot take weights");
    ModelFiles files = open_model_files(folder);
    auto decls = model.tensor_decls();
    check_names_and_shapes(decls, files.records);
    std::map<std::string, std::string> inits;
    for (auto& d : decls) inits[d.first] = d.second.init;
    Uploader up(model.rt->dev);
    model.load_tensors([&](const std::string& prefix) {
        return std::unique_ptr<TensorSource>(new FileSource(model.rt, &files.records, &inits, prefix, &up));
    });
    model.rt->dev->arena_release();        // what the conversions needed goes back to the driver
}

void init_random_weights(DecoderModel& model, unsigned long long seed) {
    if (!model.rt) throw EngineError("a model without a device cannot take weights");
    std::map<std::string, TensorDecl> decls;
    for (auto& d : model.tensor_decls()) decls[d.first] = d.second;
    model.load_tensors([&](const std::string& prefix) {
        return std::unique_ptr<TensorSource>(new RandomSource(model.rt, &decls, prefix, seed));
    });
    model.rt->dev->arena_release();
}

float random_value(unsigned long long seed, const std::string& name, long long i, const std::string& init) {
    const unsigned long long base = illm_random_base(illm_random_key(seed, name.c_str()));
    // one multiplication and one addition, each rounded once (volatile keeps the compiler from fusing them)
    volatile float scaled = (float)illm_random_centered_sum(base, (unsigned long long)i) * (0.02f / 65536.0f);
    volatile float v = scaled + (init == "norm" ? 1.0f : 0.0f);
    return v;
}

static uint16_t f32_to_f16_bits(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    const uint32_t sign = (u >> 16) & 0x8000u;
    int32_t exp = (int32_t)((u >> 23) & 0xFF) - 127 + 15;
    uint32_t man = u & 0x7FFFFFu;
    if (exp >= 31) return (uint16_t)(sign | 0x7C00u);
    if (exp <= 0) {
        if (exp < -10) return (uint16_t)sign;
        man |= 0x800000u;
        const int shift = 14 - exp;
        uint32_t half = man >> shift;
        const uint32_t rem = man & ((1u << shift) - 1), mid = 1u << (shift - 1);
        if (rem > mid || (rem == mid && (half & 1))) half++;
        return (uint16_t)(sign | half);
    }
    uint32_t half = (uint32_t)exp << 10 | man >> 13;
    const uint32_t rem = man & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) half++;
    return (uint16_t)(sign | half);
}

void write_random_model(const ArchConfig& config, const std::string& folder, unsigned long long seed, DType dtype) {
    if (dtype != DType::BF16 && dtype != DType::F32 && dtype != DType::F16)
        throw WeightError("a random model is stored as bfloat16, float32 or float16");
    mkdir(folder.c_str(), 0777);
    struct stat st;
    if (stat(folder.c_str(), &st) != 0 || !S_ISDIR(st.st_mode)) throw WeightError(folder + ": cannot be created");
    DecoderModel model(config.model_spec(), nullptr);
    auto decls = model.tensor_decls();
    Json cfg = config.to_json();
    cfg.set("torch_dtype", dtype_word(dtype));
    {
        std::ofstream f(folder + "/config.json");
        if (!f) throw WeightError(folder + "/config.json: cannot be written");
        f << cfg.dump(1) << "\n";
    }
    std::vector<TensorToWrite> tensors;
    for (auto& d : decls) tensors.push_back(TensorToWrite{d.first, d.second.init == "int" ? DType::I32 : dtype, d.second.shape});
    Json meta = Json::object();
    meta.set("format", "pt");
    meta.set("seed", std::to_string(seed));
    write_safetensors(folder + "/model.safetensors", tensors, [&](size_t idx, void* dst, size_t bytes) {
        const TensorDecl& d = decls[idx].second;
        if (d.init == "int") {
            memset(dst, 0, bytes);
            return;
        }
        const unsigned long long base = illm_random_base(illm_random_key(seed, decls[idx].first.c_str()));
        const float mean = d.init == "norm" ? 1.0f : 0.0f, scale = 0.02f / 65536.0f;
        const long long n = d.numel();
        for (long long i = 0; i < n; i++) {
            volatile float scaled = (float)illm_random_centered_sum(base, (unsigned long long)i) * scale;
            volatile float v = scaled + mean;
            const float val = v;
            if (dtype == DType::F32) ((float*)dst)[i] = val;
            else if (dtype == DType::BF16) ((uint16_t*)dst)[i] = f32_to_bf16_bits(val);
            else ((uint16_t*)dst)[i] = f32_to_f16_bits(val);
        }
    }, meta);
}

}  // namespace illm
