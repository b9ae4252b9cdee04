#pragma once
// Argument checks of CudaLlamaDecoder::create: the configuration's ranges and the shape / type of every weight the configuration implies. Which argument is
// refused with which code, and which refusal comes first when several apply, is the contract of the reference's create
// (src/backend/metal/metal_llama_decoder.mm:425-494) that its tests and callers rely on; how the checks are organized here is this backend's own: the
// expectations are laid out as a list (one entry per tensor, in contract order) and one routine judges an entry.
#include <cstdint>
#include <string>
#include <vector>

#include "cuda_llama_decoder.h"

namespace dooms {

// What a tensor has to look like.
enum class TensorRole {
    Matrix,      // a projection or the embedding table: one of the matrix types, rows of whole blocks
    Vector,      // a norm gain or a bias: f32 or f16
};

struct ExpectedTensor {
    const WeightRef * given;
    std::string name;
    int64_t rows, cols;
    TensorRole role;
};

// InvalidArgument / Unsupported for a configuration outside what the kernels handle.
Status validate_config(const LlamaDecoderConfig & c, size_t n_layer_weights);
// Every tensor the configuration implies, in the order they are checked.
Result<std::vector<ExpectedTensor>> expected_tensors(const LlamaDecoderConfig & c, const LlamaDecoderWeights & w);
Status validate_tensor(const ExpectedTensor & e);
// validate_config, then every expected tensor, then the cross-tensor rule (gate and up share a type).
Status validate_model(const LlamaDecoderConfig & c, const LlamaDecoderWeights & w);

}  // namespace dooms
