// Reader of model weight files in the safetensors layout (an 8-byte little-endian header length, a JSON header
// that maps tensor names to dtype / shape / byte range, then the raw tensor bytes).  Stands where the reference
// resolves and validates its model bundle on disk (ModelBundle::from_dir / validate_base, src/models.rs:31-104).
#pragma once
#include <stdint.h>

#include <map>
#include <string>
#include <vector>

namespace sb {

struct WeightEntry {
    std::string dtype;           // "F32", "F16" or "BF16"
    std::vector<int64_t> shape;
    uint64_t begin = 0, end = 0;  // byte range inside the data section
    int64_t numel() const {
        int64_t n = 1;
        for (int64_t d : shape) n *= d;
        return n;
    }
};

struct WeightFile {
    std::map<std::string, WeightEntry> entries;
    std::map<std::string, std::string> metadata;  // "__metadata__" of the header, if any
    std::vector<unsigned char> data;               // the data section
    // f32 view of a tensor: points into `data` for aligned F32 tensors, else into `converted`
    std::map<std::string, std::vector<float>> converted;
    const float* as_f32(const std::string& name);
};

// Returns "" on success, else a message; *missing is set when the file does not exist.
std::string weight_file_open(const char* path, WeightFile* out, bool* missing);

}  // namespace sb
