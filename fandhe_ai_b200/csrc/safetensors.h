// Parsed view of a safetensors byte buffer (safetensors.cu).
#pragma once
#include <stdint.h>

#include <string>
#include <vector>

namespace b200 {

struct StTensor {
    std::string name;
    std::string dtype;              // "F32", "I8", ...
    std::vector<uint64_t> shape;
    uint64_t begin = 0, end = 0;    // byte range inside the data buffer
    const uint8_t* data = nullptr;  // start of the tensor's bytes (little endian)
};

// Parses and validates header and layout.  On failure returns false with a message in *err.
bool safetensors_parse(const uint8_t* bytes, size_t len, std::vector<StTensor>* out, std::string* err);

}  // namespace b200
