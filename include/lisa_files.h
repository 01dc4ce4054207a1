/*
 * lisa_files — C ABI of the host-side weight-file readers that sit in front of the kernels of lisa_cuda.h:
 * the GGUF v3 container (header, tensor geometry, shards, bounded disk reads, page-aligned mappings) and
 * the safetensors shard with its {weight, scales, biases} triplets.  Plain C++ on the host, no CUDA calls;
 * exported from the same shared library.  Each comment names the reference interface the entry point
 * replaces (paths are relative to the agnosticeng/lisa repository).
 *
 * Conventions: functions return 0 on success and a negative lisa_status (lisa_cuda.h) otherwise;
 * lisa_cuda_last_error_string() describes the calling thread's last failure, with the reference's own
 * messages ("invalid GGUF magic", "only GGUF version 3 is supported", "overlapping GGUF tensors ...").
 * Handles are owned by the caller and closed with the matching *_close.  Strings returned by accessors
 * live as long as the handle.  Nothing here reads a tensor payload unless asked to (read_*, map_*).
 */
#ifndef LISA_FILES_H
#define LISA_FILES_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---------------------------------------------------------------- GGUF block geometry
 * TensorType::layout / TensorType::row_bytes, crates/lisa-gguf/src/lib.rs:35-83.
 * layout: name, elements per block, bytes per block of a GGML type id; LISA_ERR_UNSUPPORTED for an id the
 * table does not hold.  row_bytes: bytes of a row of `columns` elements; columns must be a positive multiple
 * of the block. */
int lisa_gguf_type_layout(uint32_t type, const char **name, uint64_t *block_elements, uint64_t *block_bytes);
int lisa_gguf_row_bytes(uint32_t type, uint64_t columns, uint64_t *row_bytes);

/* ---------------------------------------------------------------- GGUF header and package */
typedef struct lisa_gguf lisa_gguf;

typedef struct lisa_gguf_tensor {
    const char *name;
    uint32_t rank;          /* 1..4 */
    uint64_t dimensions[4]; /* GGML order: contiguous input columns first, then rows, then experts */
    uint32_t type;          /* GGML type id */
    uint64_t offset;        /* absolute byte offset of the payload in its shard file */
    uint64_t bytes;
    uint64_t rows;          /* product of dimensions[1..] */
    uint64_t row_bytes;
    int32_t shard;          /* index into the package's shard list */
} lisa_gguf_tensor;

/* Header::read, crates/lisa-gguf/src/header.rs:110-214: parses a header held in memory.  `file_bytes` is
 * the length of the complete file, which may exceed `length` (a bounded download of the header can be
 * inspected before the weights are fetched); every tensor range is checked against it.  All of the
 * reference's checks: magic, version 3, entry limits, key and name rules, alignment (general.alignment,
 * default 32, a power of two <= 65536), rank 1..4, non-zero dimensions, overflow, type geometry, aligned
 * offsets, ranges inside the file, no overlap, no duplicates, no nested arrays. */
int lisa_gguf_parse(const void *bytes, uint64_t length, uint64_t file_bytes, lisa_gguf **out);
/* Package::open, crates/lisa-gguf/src/package.rs:162-217: opens a file and, when split.count > 1, the other
 * shards named `<stem>-000NN-of-000MM.gguf` beside it (the first shard must be given; split.no /
 * split.count / split.tensors.count and the architecture must agree; tensor names must be unique across
 * shards).  The DeepSeek Engram side file of package.rs:199-213 is not looked for. */
int lisa_gguf_open(const char *path, lisa_gguf **out);
/* Package::open_paths, package.rs:220-292: an explicit shard list. */
int lisa_gguf_open_paths(const char *const *paths, int count, lisa_gguf **out);
void lisa_gguf_close(lisa_gguf *g);

uint64_t lisa_gguf_data_offset(const lisa_gguf *g); /* of the first shard */
uint64_t lisa_gguf_file_bytes(const lisa_gguf *g);
int lisa_gguf_shard_count(const lisa_gguf *g);
const char *lisa_gguf_shard_path(const lisa_gguf *g, int shard); /* NULL for a parsed buffer */
int64_t lisa_gguf_tensor_count(const lisa_gguf *g);
/* Tensors are held sorted by name (the reference keeps them in a BTreeMap). */
int lisa_gguf_tensor_at(const lisa_gguf *g, int64_t index, lisa_gguf_tensor *out);
/* Package::tensor, package.rs:294-298: index of `name`, or LISA_ERR_BAD_ARG ("missing GGUF tensor ..."). */
int64_t lisa_gguf_find_tensor(const lisa_gguf *g, const char *name);

/* Metadata of the first shard.  Header::integer / Header::architecture, header.rs:216-229, and
 * Value::{as_u64, as_f64, as_str, as_array}, header.rs:24-56.
 * kind: 0 unsigned, 1 signed, 2 float, 3 bool, 4 string, 5 array; -1 when the key is absent. */
int lisa_gguf_metadata_kind(const lisa_gguf *g, const char *key);
int lisa_gguf_metadata_u64(const lisa_gguf *g, const char *key, uint64_t *out);
int lisa_gguf_metadata_f64(const lisa_gguf *g, const char *key, double *out);
const char *lisa_gguf_metadata_str(const lisa_gguf *g, const char *key); /* NULL when absent or not a string */
int64_t lisa_gguf_metadata_array_len(const lisa_gguf *g, const char *key); /* -1 when absent or not an array */
int lisa_gguf_metadata_array_u64(const lisa_gguf *g, const char *key, int64_t index, uint64_t *out);
const char *lisa_gguf_metadata_array_str(const lisa_gguf *g, const char *key, int64_t index);

/* Tensor::read_bytes / Tensor::read_rows, package.rs:112-156: positional reads bounded to 64 MiB per call
 * and to the tensor's own range; rows are delivered in caller order. */
int lisa_gguf_read_bytes(const lisa_gguf *g, int64_t tensor, uint64_t offset, void *out, uint64_t length);
int lisa_gguf_read_rows(const lisa_gguf *g, int64_t tensor, const uint64_t *rows, uint64_t count, void *out,
                        uint64_t out_bytes);
/* Tensor::mapped_region_bytes / mapped_region, package.rs:26-66: a read-only mapping of the pages that hold
 * the tensor; *inner is the tensor's byte offset inside the mapping.  lisa_gguf_unmap releases it; the
 * mapping outlives lisa_gguf_close. */
int lisa_gguf_mapped_region_bytes(const lisa_gguf *g, int64_t tensor, uint64_t *bytes);
int lisa_gguf_map_region(const lisa_gguf *g, int64_t tensor, void **mapping, uint64_t *mapped_bytes, uint64_t *inner);
int lisa_gguf_unmap(void *mapping, uint64_t mapped_bytes);
/* The view the engine gives the kernels, crates/lisa-engine/src/core/gguf_resident.rs:95-101: dimensions
 * after the first reversed, row_bytes appended: uint8 [experts, rows, row_bytes] (experts = 1 for a matrix;
 * a rank-4 tensor folds its two outer dimensions into experts).  These are the arguments of
 * lisa_cuda_gguf_packed_matvec / lisa_cuda_gguf_expert_matvec. */
int lisa_gguf_weight_view(const lisa_gguf *g, int64_t tensor, int64_t *experts, int64_t *rows, int64_t *row_bytes);

/* ---------------------------------------------------------------- safetensors shard
 * Shard::open / tensor_bytes / tensor_names, crates/lisa-engine/src/core/loader.rs:57-160: the file is
 * mapped read-only, the JSON header (<= 64 MiB) is parsed, every tensor's range is checked against the
 * payload and against its shape. */
typedef struct lisa_safetensors lisa_safetensors;

/* dtype codes: the reference's accepted set (loader.rs:88-98). */
typedef enum lisa_st_dtype {
    LISA_ST_BF16 = 0, LISA_ST_F32 = 1, LISA_ST_F16 = 2, LISA_ST_I64 = 3, LISA_ST_I32 = 4, LISA_ST_U32 = 5,
    LISA_ST_U8 = 6, LISA_ST_BOOL = 7
} lisa_st_dtype;

typedef struct lisa_st_tensor {
    const char *name;
    int32_t dtype; /* lisa_st_dtype */
    int32_t rank;  /* <= 8 */
    int64_t shape[8];
    const void *data; /* inside the shard's mapping */
    uint64_t bytes;
} lisa_st_tensor;

int lisa_safetensors_open(const char *path, lisa_safetensors **out);
void lisa_safetensors_close(lisa_safetensors *s);
int64_t lisa_safetensors_tensor_count(const lisa_safetensors *s);
int lisa_safetensors_tensor_at(const lisa_safetensors *s, int64_t index, lisa_st_tensor *out); /* sorted by name */
int lisa_safetensors_find(const lisa_safetensors *s, const char *name, lisa_st_tensor *out);

/* detect_group_size, crates/lisa-engine/src/core/quant.rs:273-287: the group size implied by the packed
 * shapes, or 0 when they are inconsistent. */
int32_t lisa_detect_group_size(int32_t weight_cols, int32_t scales_cols, int32_t bits);

/* QuantizedLinear::load / QuantizedEmbedding::load, quant.rs:408-432,474-491: the triplet
 * `{prefix}.{key}.weight/.scales/.biases` (key may be empty or NULL: `{prefix}.weight` ...), with the group
 * size detected from the shapes for `bits` (fallback `group_size_hint`).  weight must be U32 [N, K*bits/32],
 * scales and biases the same 16-bit float type [N, K/group]. */
typedef struct lisa_quantized_triplet {
    lisa_st_tensor weight, scales, biases;
    int32_t group_size, bits;
    int64_t n, k;
} lisa_quantized_triplet;
int lisa_safetensors_quantized_triplet(const lisa_safetensors *s, const char *prefix, const char *key, int32_t bits,
                                       int32_t group_size_hint, lisa_quantized_triplet *out);

#ifdef __cplusplus
}
#endif
#endif
