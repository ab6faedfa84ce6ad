// Loading a model's tensors from safetensors by name, random weights, and writing a random model folder.
//
// The reference looks tensors up by name as well, after translating the file's names through an
// alias table (src/graph/llama_like.cpp:9-22, src/core/graph.cpp:233-257); an unknown tensor is
// skipped with a log line (:311-317), a wrong size aborts (:322-326) and a tensor that the file lacks
// goes unnoticed (src/core/tensor.cpp:57-59).  Here the model declares every tensor it needs under
// the file's own names, and one error lists all that is missing, unexpected or of the wrong shape
// before anything is copied.
//
// Storage rule: floating-point tensors stored in 16 bits are kept in bfloat16, a tensor stored in
// 32-bit stays so, integer tables become int32; in the float32 mode every floating-point tensor is
// widened to float32.  Matrices are then brought to the compute dtype by the part that owns them.
//
// Random weights: matrices N(0, 0.02), norm weights 1 + N(0, 0.02), each from the stream of (seed,
// tensor name), so a tensor does not depend on which others exist.  The numbers are defined bit by
// bit (csrc/random_init.h): filled on the device by a kernel or made on the host for a model folder,
// the same seed gives the same tensors.
#pragma once
#include <map>
#include <string>
#include <vector>

#include "models/decoder.h"
#include "weights/safetensors.h"

namespace illm {

// WeightError listing every missing tensor, every unexpected one (derived tables that some exporters
// store, "rotary_emb.inv_freq", are tolerated) and every wrong shape.
void check_names_and_shapes(const std::vector<std::pair<std::string, TensorDecl>>& decls,
                            const std::map<std::string, TensorRecord>& records);
DType storage_dtype(DType stored, DType runtime_dtype, const std::string& init);

// Check the folder's tensors against the model's declarations (no device needed).
void check_model_folder(const DecoderModel& model, const std::string& folder);
// ... and hand them to the parts (the model was built on a device).
void load_model_weights(DecoderModel& model, const std::string& folder);
// Fill a model on its device with random weights without going through a file (for sizes where
// writing and reading tens of gigabytes would only cost time).
void init_random_weights(DecoderModel& model, unsigned long long seed);
// Write config.json and model.safetensors with random weights for a typed configuration; `dtype`
// is the stored dtype of every tensor (bfloat16, float32 or float16).
void write_random_model(const ArchConfig& config, const std::string& folder, unsigned long long seed, DType dtype);
// Element i of the random tensor `name` as float32 (the host twin of the fill kernel).
float random_value(unsigned long long seed, const std::string& name, long long i, const std::string& init);

}  // namespace illm
