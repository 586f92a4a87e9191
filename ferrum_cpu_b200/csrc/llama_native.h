// Internal: what the GGUF reader hands to the decoder when the matrices are to stay in their file format.
#pragma once
#include <cstddef>
#include <cstdint>

#include "../../include/ferrum_cuda.h"

namespace fc {

struct RawTensor {          // one matrix [n_out][n_in] as stored in the file
    int type = -1;          // ggml type
    const uint8_t* data = nullptr;
    size_t nbytes = 0;
};
struct RawLlamaLayer { RawTensor wq, wk, wv, wo, gate, up, down; };

// fc_llama_create with the matrices uploaded in their own block formats (native footprint) instead of as Q8_0: `w`
// supplies the f32 vectors (norms, biases, RoPE factors); tok / output / layers the matrices (output.data null: tied head).
int llama_create_native(const fc_llama_config* cfg, const fc_llama_weights* w, const RawTensor& tok, const RawTensor& output,
                        const RawLlamaLayer* layers, int device, fc_llama** out);

}  // namespace fc
