// safetensors.h — a memory-mapped .safetensors file: header parsed on the host, tensor bytes
// left where the page cache has them until an upload copies them to the device.
// (What catgrad-llm/examples/llama/main.rs:296-330 does through the safetensors and memmap2
// crates: 8-byte little-endian header length, a JSON object name -> {dtype, shape,
// data_offsets}, then the raw little-endian tensor bytes.)
#pragma once

#include <cstdint>
#include <string>
#include <vector>

#include "runtime.h"

namespace cg {

struct StEntry {
  std::string name;
  int storage = ST_F32;        // ST_F32 or ST_BF16 (the two dtypes the reference's loader accepts)
  std::vector<int64_t> dims;
  size_t begin = 0, end = 0;   // byte range inside the data section
  int64_t numel() const {
    int64_t n = 1;
    for (int64_t d : dims) n *= d;
    return n;
  }
};

}  // namespace cg

struct cg_safetensors {
  std::string path;
  void* map = nullptr;         // whole file, read-only
  size_t map_bytes = 0;
  const uint8_t* data = nullptr;  // start of the data section
  size_t data_bytes = 0;
  std::vector<cg::StEntry> entries;  // in header order, "__metadata__" dropped
  ~cg_safetensors();
};

namespace cg {

// Opens and parses; on failure returns null and says why.
cg_safetensors* st_open(const char* path, std::string* why);
// Uploads entry `e` as a tensor of context c.  With keep_bf16 (a bf16-precision context and a
// rank >= 2 tensor) bf16 bytes go to the device as they are; otherwise the result is f32
// (bf16 sources are widened on the device, never on the host).
int st_upload(cg_ctx* c, const cg_safetensors* f, const StEntry& e, cg_tensor** out);
// Copies entry `e` into dst (bf16 storage, contiguous) at element offset `at`, converting f32
// sources on the device.
int st_upload_into_bf16(cg_ctx* c, const cg_safetensors* f, const StEntry& e, cg_tensor* dst, int64_t at);

}  // namespace cg
