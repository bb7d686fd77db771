/* GGUF model-file reader and packed-weight upload: C ABI of librunit_cuda.so.
 *
 * Replaces, for the quantized decode path, the reference's `bare-metal-gguf` crate and the upload half of its engine:
 *   crates/gguf/src/parser.rs:22-57      GgufParser::parse (header, metadata KV pairs, tensor index, aligned data offset)
 *   crates/gguf/src/parser.rs:229        parse_gguf_file(path)
 *   crates/gguf/src/types.rs:18-63       GgufFile / GgufTensorInfo (num_elements, data_size)
 *   crates/gguf/src/types.rs:69-199      GgufDtype: ggml type ids, block_size, type_size, tensor_data_size
 *   crates/gguf/src/types.rs:241-336     GgufMetadataValueType / GgufMetadataValue accessors
 *   crates/gguf/src/error.rs:4-31        GgufError kinds (one status code each, same message texts)
 *   crates/engine/src/forward.rs:1137-1222, 1321-1418   weight upload: here the Q8_0 / Q4_0 / Q4_K bytes go to device memory
 *       exactly as they sit in the file (the fused-dequant kernels read the packed blocks), and a merged expert tensor
 *       `blk.N.ffn_{gate,up,down}_exps.weight` ([K, rows, E] in file order = [E][rows][K/256 * 144 B]) stays one buffer with
 *       expert e at byte e * rows * row_bytes -- the layout the MoE entry points of runit_cuda.h take.
 *
 * Parsing needs no GPU.  Handles are not thread-safe; error texts are per thread (runit_gguf_last_error).
 */
#ifndef RUNIT_GGUF_H
#define RUNIT_GGUF_H

#include <stddef.h>
#include <stdint.h>

#include "runit_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif

/* crates/gguf/src/types.rs:6-13 */
#define RUNIT_GGUF_MAGIC 0x46554747u
#define RUNIT_GGUF_DEFAULT_ALIGNMENT 32u

/* status codes: crates/gguf/src/error.rs:4-31, plus lookups and argument checks of this ABI */
enum {
    RUNIT_GGUF_OK = 0,
    RUNIT_GGUF_ERR_IO = 1,
    RUNIT_GGUF_ERR_INVALID_MAGIC = 2,
    RUNIT_GGUF_ERR_UNSUPPORTED_VERSION = 3,
    RUNIT_GGUF_ERR_UNKNOWN_DTYPE = 4,
    RUNIT_GGUF_ERR_UNKNOWN_METADATA_TYPE = 5,
    RUNIT_GGUF_ERR_UNEXPECTED_EOF = 6,
    RUNIT_GGUF_ERR_INVALID_UTF8 = 7,
    RUNIT_GGUF_ERR_DATA_REGION_OVERFLOW = 8,
    RUNIT_GGUF_ERR_NOT_FOUND = 9,      /* no tensor / metadata key of that name, or the value has another type */
    RUNIT_GGUF_ERR_BAD_ARG = 10,
    RUNIT_GGUF_ERR_BUFFER_SIZE = 11,   /* destination smaller than the tensor */
    RUNIT_GGUF_ERR_CUDA = 12
};

/* ggml type ids handled by the kernels (crates/gguf/src/types.rs:69-100 lists all of them) */
#define RUNIT_GGUF_TYPE_F32 0u
#define RUNIT_GGUF_TYPE_F16 1u
#define RUNIT_GGUF_TYPE_Q4_0 2u
#define RUNIT_GGUF_TYPE_Q8_0 8u
#define RUNIT_GGUF_TYPE_Q4_K 12u

/* metadata value types: crates/gguf/src/types.rs:241-256 */
enum {
    RUNIT_GGUF_META_UINT8 = 0, RUNIT_GGUF_META_INT8 = 1, RUNIT_GGUF_META_UINT16 = 2, RUNIT_GGUF_META_INT16 = 3,
    RUNIT_GGUF_META_UINT32 = 4, RUNIT_GGUF_META_INT32 = 5, RUNIT_GGUF_META_FLOAT32 = 6, RUNIT_GGUF_META_BOOL = 7,
    RUNIT_GGUF_META_STRING = 8, RUNIT_GGUF_META_ARRAY = 9, RUNIT_GGUF_META_UINT64 = 10, RUNIT_GGUF_META_INT64 = 11,
    RUNIT_GGUF_META_FLOAT64 = 12
};

typedef struct runit_gguf runit_gguf_t;

/* GgufTensorInfo (crates/gguf/src/types.rs:41-63).  ne[] are the dimensions in file order: ne[0] is the row length K. */
typedef struct runit_gguf_tensor_info {
    const char* name;        /* owned by the handle */
    uint32_t dtype;          /* ggml type id */
    uint32_t n_dims;
    uint64_t ne[4];
    uint64_t data_offset;    /* relative to runit_gguf_data_offset() */
    uint64_t num_elements;   /* product of ne, at least 1 */
    uint64_t data_size;      /* bytes: ceil(num_elements / block_size) * type_size */
} runit_gguf_tensor_info;

/* parse_gguf_file / GgufParser::parse.  open_memory parses a caller-owned image that must outlive the handle. */
int32_t runit_gguf_open(const char* path, runit_gguf_t** out);
int32_t runit_gguf_open_memory(const void* image, uint64_t bytes, runit_gguf_t** out);
void runit_gguf_close(runit_gguf_t* g);
const char* runit_gguf_last_error(void);

uint32_t runit_gguf_version(const runit_gguf_t* g);
uint64_t runit_gguf_alignment(const runit_gguf_t* g);     /* `general.alignment`, default 32 */
uint64_t runit_gguf_data_offset(const runit_gguf_t* g);   /* absolute offset of the tensor data region */
uint64_t runit_gguf_tensor_count(const runit_gguf_t* g);
uint64_t runit_gguf_metadata_count(const runit_gguf_t* g);

int32_t runit_gguf_tensor_at(const runit_gguf_t* g, uint64_t index, runit_gguf_tensor_info* out);
int32_t runit_gguf_tensor_find(const runit_gguf_t* g, const char* name, runit_gguf_tensor_info* out);

/* GgufDtype::{block_size, type_size, tensor_data_size, Display}; 0 / NULL for an unknown type id */
uint64_t runit_gguf_dtype_block_size(uint32_t dtype);
uint64_t runit_gguf_dtype_type_size(uint32_t dtype);
uint64_t runit_gguf_dtype_tensor_data_size(uint32_t dtype, uint64_t num_elements);
const char* runit_gguf_dtype_name(uint32_t dtype);

/* Metadata.  key_at enumerates keys in file order; type reports the value type (for arrays also the element type and
 * count).  The scalar getters widen (as_u32 / as_u64 / as_f32 of the reference accept exactly one type each; these
 * accept every integer type (and bool as 0 / 1) for u64 / i64 and both float widths for f64, and report NOT_FOUND
 * otherwise). */
int32_t runit_gguf_meta_key_at(const runit_gguf_t* g, uint64_t index, const char** key);
int32_t runit_gguf_meta_type(const runit_gguf_t* g, const char* key, uint32_t* type, uint32_t* elem_type, uint64_t* count);
int32_t runit_gguf_meta_u64(const runit_gguf_t* g, const char* key, uint64_t* out);
int32_t runit_gguf_meta_i64(const runit_gguf_t* g, const char* key, int64_t* out);
int32_t runit_gguf_meta_f64(const runit_gguf_t* g, const char* key, double* out);
int32_t runit_gguf_meta_bool(const runit_gguf_t* g, const char* key, int32_t* out);
int32_t runit_gguf_meta_str(const runit_gguf_t* g, const char* key, const char** out, uint64_t* len);
int32_t runit_gguf_meta_array_u64(const runit_gguf_t* g, const char* key, uint64_t index, uint64_t* out);
int32_t runit_gguf_meta_array_i64(const runit_gguf_t* g, const char* key, uint64_t index, int64_t* out);
int32_t runit_gguf_meta_array_f64(const runit_gguf_t* g, const char* key, uint64_t index, double* out);
int32_t runit_gguf_meta_array_str(const runit_gguf_t* g, const char* key, uint64_t index, const char** out, uint64_t* len);

/* Tensor bytes as stored in the file, into host memory. */
int32_t runit_gguf_read_tensor(runit_gguf_t* g, const char* name, void* host_dst, uint64_t capacity);
/* Tensor bytes as stored in the file, into device memory, ordered on the context's stream (two pinned staging buffers:
 * the file read of one chunk overlaps the copy of the previous one).  Returns after the last copy was enqueued and the
 * staging buffers are free again; the data is visible to later launches of the context. */
int32_t runit_gguf_upload_tensor(runit_ctx_t* ctx, runit_gguf_t* g, const char* name, void* device_dst, uint64_t capacity);

#ifdef __cplusplus
}
#endif

#endif /* RUNIT_GGUF_H */
