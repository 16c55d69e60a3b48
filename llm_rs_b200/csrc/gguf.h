// GGUF container reader: header, metadata and tensor directory of a v2 / v3 file, and positional
// reads of tensor bytes.  Counterpart of src/gguf/mod.rs (GgufFile::open :167-218, tensor_view
// :242-254, metadata values :256-303, read_file_fast :307-342) for a machine whose weights live in
// device memory: only the directory is kept on the host; tensor bytes go from the file through
// pinned staging buffers to the GPU (backend.cu) instead of being held in one page-aligned copy
// of the whole file.
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <string_view>
#include <vector>

namespace llmrs {

// Value types of the metadata section (src/gguf/mod.rs:256-273).
enum GgufType : uint32_t {
    GT_U8 = 0, GT_I8 = 1, GT_U16 = 2, GT_I16 = 3, GT_U32 = 4, GT_I32 = 5, GT_F32 = 6, GT_BOOL = 7,
    GT_STRING = 8, GT_ARRAY = 9, GT_U64 = 10, GT_I64 = 11, GT_F64 = 12
};

struct GgufValue {
    std::string key;
    uint32_t type = 0;            // GgufType
    uint32_t elem_type = 0;       // arrays: type of the elements
    uint64_t count = 0;           // arrays: number of elements
    // scalars: the value widened (integers and bool in u, floats in f); strings: s
    uint64_t u = 0;
    double f = 0.0;
    std::string_view s;                       // borrowed from the header bytes
    size_t data_pos = 0;                      // numeric arrays: position of the packed little-endian elements
    std::vector<std::string_view> strings;    // string arrays
};

struct GgufTensor {
    std::string name;
    uint32_t dtype = 0;           // GGUF type id (src/tensor/mod.rs:96-130)
    uint32_t n_dims = 0;
    uint64_t shape[4] = {0, 0, 0, 0};
    uint64_t offset = 0;          // relative to the data section
    uint64_t nbytes = 0;          // storage size of the shape in this dtype
};

// Elements per block and bytes per block of a GGUF dtype id; false for ids the format does not define
// (src/tensor/mod.rs:36-93).
bool gguf_block_layout(uint32_t dtype, uint32_t *block_elems, uint32_t *block_bytes);

struct GgufFile {
    int fd = -1;
    uint64_t file_size = 0;
    uint32_t version = 0;
    uint64_t data_offset = 0;     // first byte of the tensor data: header end rounded up to 32
    std::vector<uint8_t> header;  // the bytes up to data_offset (strings above borrow from it)
    std::vector<GgufValue> metadata;
    std::vector<GgufTensor> tensors;

    ~GgufFile();
    const GgufValue *find_value(const char *key) const;
    const GgufTensor *find_tensor(const char *name) const;
};

// Opens and parses `path`.  On failure returns nullptr and writes a message to *error.
GgufFile *gguf_open(const char *path, std::string *error);

// Reads file bytes [offset, offset + len) into dst with `threads` concurrent positional reads over
// equal stripes, each in pieces of 4 MiB (src/gguf/mod.rs:307-342).  False on a short or failed read.
bool gguf_pread_parallel(int fd, void *dst, uint64_t offset, size_t len, int threads);

}  // namespace llmrs
