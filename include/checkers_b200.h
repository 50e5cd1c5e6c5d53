/*
 * checkers_b200.h -- C ABI of the B200 checkpoint-compression library
 * (libcheckers_b200.so).
 *
 * The Checkers reference exposes this path as three pybind11 functions backed
 * by a process-wide registry; it has no C ABI.  Each entry point below names
 * the reference interface it stands in for (file:line inside the Checkers
 * tree), so a binding for the reference's own front end can be written one to
 * one.  Plain pointers and sizes only; no exceptions cross this boundary:
 * every function returns CHK_OK (0) or a negative CHK_ERR_* code and leaves a
 * message for chk_last_error() on the calling thread.
 *
 * Tensors are BORROWED device pointers, exactly as in the reference
 * (src/TensorResource.cpp:16-33): they must stay valid and unchanged from
 * registration until the call that uses them returns.  All work of a context
 * is issued on the device given at creation; a context is not thread-safe.
 */
#ifndef CHECKERS_B200_H
#define CHECKERS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CHK_OK 0
#define CHK_ERR_INVALID (-1)  /* bad argument or call order */
#define CHK_ERR_CUDA (-2)     /* a CUDA runtime call failed */
#define CHK_ERR_IO (-3)       /* file could not be read or written */
#define CHK_ERR_FORMAT (-4)   /* file contents are not a valid checkpoint */
#define CHK_ERR_DECODE (-5)   /* a stream failed its end-state / length check */
#define CHK_ERR_UNDECODABLE (-6) /* shared tables that do not sum to 4096: the files could not be restored */
#define CHK_ERR_CAPACITY (-7) /* a size exceeds a stated fixed limit */

/* DataType tags, include/checkers/TensorResource.hpp:30-37 */
enum { CHK_F32 = 0, CHK_BF16 = 1, CHK_F16 = 2, CHK_I8 = 3, CHK_I32 = 4, CHK_DTYPE_UNKNOWN = 255 };
/* TensorCategory tags, include/checkers/TensorResource.hpp:59-65 */
enum { CHK_CAT_MODEL = 0, CHK_CAT_MASTER = 1, CHK_CAT_EXP_AVG = 2, CHK_CAT_EXP_AVG_SQ = 3, CHK_CAT_UNKNOWN = 255 };

typedef struct chk_context chk_context;

/* Per-rank totals of the last compression; the six numbers every rank
 * contributes to the all-gathered manifest. */
typedef struct {
    uint64_t n_tensors;
    uint64_t n_tables;
    uint64_t states_bytes;   /* size of rank_<r>_states.ansc */
    uint64_t mantissa_bytes; /* size of rank_<r>_mantissa.mant */
    uint64_t dict_bytes;     /* size of rank_<r>_tables.dict */
    uint64_t original_bytes; /* uncompressed bytes of the tensors written */
} chk_summary;

const char* chk_last_error(void);

/* ---- context and registry ------------------------------------------------
 * chk_context_create + chk_register_tensor replace
 * checkers::initialize_context (src/api.cpp:899-1031) minus its DeepSpeed
 * object walk: the caller hands over what that walk would have found
 * (name, device pointer, element count, dtype; src/api.cpp:789-850,
 * MemoryManager::submit_tensor src/MemoryManager.cpp:218-250).  Records keep
 * submission order, which is the order of every output file. */
int chk_context_create(int device, int rank, int local_rank, chk_context** out);
/* The same with a bound on the context's encode workspace (the reference sizes its buffers per tensor,
 * src/ANSCompressor.cpp:348-388, and its statistics slabs per batch, src/MemoryManager.cpp:692-707; here the
 * one pool that grows with the work is the encoder's scratch).  Compression keeps one scratch slot -- twice
 * the largest tensor's codec input, the worst case of its 256 lanes -- per resident encode team; with
 * workspace_bytes > 0 fewer teams run so that their slots fit (slower, same bytes); a bound smaller than
 * one slot makes chk_compress return CHK_ERR_CAPACITY.  0 = no bound: one slot for every team the device
 * can hold (about 7.5 GB on a B200 for tensors of 4 MiB).  The compressed outputs -- the sidecar section
 * and the payload heap, sized for the worst case of one byte per input byte -- are not workspace. */
int chk_context_create_ex(int device, int rank, int local_rank, uint64_t workspace_bytes, chk_context** out);
int chk_context_destroy(chk_context* ctx);
int chk_reset(chk_context* ctx); /* MemoryManager::reset: forget tensors, clusters, results */
/* Gives the context's device memory (sidecar section, payload heap, encode workspace, tables, ...) back to
 * the device.  The buffers are otherwise kept from call to call and only grow; a checkpoint hook calls this
 * after a save so that the training step gets the memory back.  The device-resident result of the last
 * chk_compress is gone afterwards; host images and registered tensors stay.  (The reference frees its
 * per-tensor buffers after every tensor: src/ANSCompressor.cpp:348-388.) */
int chk_release_workspace(chk_context* ctx);
int chk_set_histogram_bins(chk_context* ctx, uint32_t bins); /* initialize_context(histogram_bins=) */
int chk_register_tensor(chk_context* ctx, const char* name, const void* device_ptr, uint64_t num_elements,
                        uint8_t dtype, uint8_t category);
int chk_tensor_count(chk_context* ctx, uint64_t* count);
/* Options: "repair_tables" (0/1; shared tables are renormalised until they sum
 * to 4096 -- a deviation from the reference that keeps them decodable),
 * "allow_undecodable" (0/1; see chk_compress_and_save), "verify_zero_lanes" (0/1;
 * decode also checks the lanes that only carry zeroed low bytes),
 * "workspace_bytes" (bound on the encode scratch, as in chk_context_create_ex),
 * "segments" (1..8, default 4: launches the counting of a batch of 512 tensors or
 * more is cut into, so that the tables of one piece are built while the next is
 * counted), "encode_teams_per_sm" / "decode_teams_per_sm" (default 0 = as many as
 * fit: cap on the resident teams per SM), "decode_zero_skip" (0/1; float tensors
 * are decoded with a slot table that leaves out the slots of the zeroed low bytes, 8.5 KiB instead of 16 KiB).  None of the tuning options changes the bytes
 * that are produced.
 * "fast_stats" (0/1, default 0): chk_analyze sums in double over tiles spread over the
 * whole device instead of in the reference's order of float additions: minimum,
 * maximum and value histogram are unchanged, mean / variance / skewness / kurtosis
 * differ by the rounding error of the reference's float sums (and cluster boundaries
 * that hang on that error can move).
 * "format_version" (2 or 3, default 2).  2 is the reference's container.  3 is an
 * experiment the reference has no counterpart for: every high byte of a
 * floating-point element becomes a byte plane that is coded as an 8-bit tensor of its
 * own ("<name>#b<byte>") with its own table, by the same coder; low bytes stay raw.
 * The three files keep their layouts and carry version 3 in their headers; a context
 * reads only the version it is set to.  Cluster-shared tables are not used.
 * "v3_fused_decode" (0/1, default 1): version-3 restore of float-only state decodes the planes straight into
 * whole elements; 0 = planes to memory, then a merge pass (the route state with integer tensors always takes). */
int chk_set_option(chk_context* ctx, const char* key, int64_t value);

/* ---- analysis: checkers::analyze_tensors, src/api.cpp:1033-1253 ----------
 * tensor_stats_kernel (src/TensorAnalyzer.cpp:64-229), fingerprints
 * (:271-292) and the per-category union-find clustering (:440-598). */
int chk_analyze(chk_context* ctx);
int chk_get_tensor_stats(chk_context* ctx, uint64_t index, uint32_t hist[256], float moments[4], float minmax[2],
                         float fingerprint[5]);
/* ---- vocabulary sketches: the reference's offline study of shared histograms
 * (scripts/llama-3-8b/experiment_2.py:31-85, 122-145: HyperLogLog with 2^14 registers over a tensor's 32-bit
 * symbols, union of a cluster = element-wise maximum).  chk_hll_sketch_all sketches every registered tensor
 * in one pass on the device; merge and count are host arithmetic on 16 KiB.  chk_shared_vocabulary_report
 * prices per-tensor histograms against histograms shared inside the current clusters (8 bytes per distinct
 * symbol + 64, as the study does). */
int chk_hll_sketch_all(chk_context* ctx);
int chk_hll_get(chk_context* ctx, uint64_t index, uint8_t regs[16384]);
int chk_hll_merge(uint8_t acc[16384], const uint8_t other[16384]);
int chk_hll_count(const uint8_t regs[16384], double* estimate);
int chk_shared_vocabulary_report(chk_context* ctx, uint64_t* per_tensor_bytes, uint64_t* shared_bytes);
/* The reference's second study (scripts/llama-3-8b/experiment_2_1.py:52-75, 217-330): the registered tensors
 * index[0..n) coded under ONE model over their 32-bit symbols -- counts quantised to a power-of-two scale, every
 * occurrence costs log2(scale / norm[symbol]) bits.  Returns the stream bytes and the size of the shared
 * vocabulary (the model costs 8 bytes per entry); a group of one tensor gives the tensor's own-model figures. */
int chk_shared_model_cost(chk_context* ctx, const uint64_t* index, uint64_t n, double* stream_bytes,
                          uint64_t* vocabulary);
/* cluster_id[i] for every registered tensor (-1 = singleton); *n_clusters out. */
int chk_get_cluster_ids(chk_context* ctx, int32_t* cluster_id, uint64_t capacity, int32_t* n_clusters);
int chk_get_cluster_anchor(chk_context* ctx, int32_t cluster, char name_out[256]);
/* MemoryManager::set_cluster_info (include/checkers/MemoryManager.hpp:180):
 * install a cluster map from outside.  ids[i] < 0 marks names[i] a singleton. */
int chk_set_cluster_info(chk_context* ctx, uint64_t n, const char* const* names, const int32_t* ids,
                         int32_t n_clusters, const char* const* anchor_names);

/* ---- codec: checkers::compress_and_save, src/api.cpp:1255-1299 -----------
 * ANSCompressor::compress_and_save_all (src/ANSCompressor.cpp:1014-1401):
 * writes <dir>/rank_<r>_states.ansc, <dir>/mantissa/rank_<r>_mantissa.mant and
 * <dir>/tables/rank_<r>_tables.dict in the reference's layout (:751-931). */
int chk_compress_and_save(chk_context* ctx, const char* output_dir);
/* Tables of the last compression and how many of them do not sum to 4096.  The reference builds the
 * table a cluster shares over the full alphabet and takes the surplus back in a single pass
 * (src/ANSCompressor.cpp:477-482); for low-entropy data (every bf16 tensor) the sum stays above 4096,
 * the streams are not decodable, and the reference itself writes past its decode arrays (:495-499).
 * Such files are reproduced bit for bit on request, but never silently: chk_compress_and_save returns
 * CHK_ERR_UNDECODABLE before writing anything unless "allow_undecodable" is set (reference-exact bytes) --
 * or "repair_tables" makes the tables valid.  Without clusters (no chk_analyze / chk_set_cluster_info)
 * every tensor owns its table and the case cannot arise. */
int chk_get_table_report(chk_context* ctx, uint64_t* n_tables, uint64_t* n_undecodable);
/* Same pipeline, results kept in memory.  host_images != 0 also builds the
 * three file images in pinned host memory (fetch with chk_get_image);
 * otherwise the compressed state stays on the device for chk_decompress_resident. */
int chk_compress(chk_context* ctx, int host_images);
/* which: 0 states, 1 mantissa, 2 tables.  Pointers stay valid until the next
 * compress call on this context. */
int chk_get_image(chk_context* ctx, int which, const void** data, uint64_t* size);
int chk_get_summary(chk_context* ctx, chk_summary* out);

/* ---- restore (the reference ships no reader; inverse of the above) -------
 * Every tensor found in the files whose name is registered in this context is
 * decoded into the registered pointer (size and dtype must match). */
int chk_load_and_decompress(chk_context* ctx, const char* input_dir);
int chk_decompress_images(chk_context* ctx, const void* states, uint64_t states_size, const void* mantissa,
                          uint64_t mantissa_size, const void* tables, uint64_t tables_size);
/* Decode the device-resident result of the last chk_compress.  dst[i] (device
 * pointer, one per registered tensor, may be NULL to skip) receives tensor i;
 * dst == NULL restores into the registered pointers. */
int chk_decompress_resident(chk_context* ctx, void* const* dst);
/* Number of tensors restored by the last decompress call. */
int chk_restored_count(chk_context* ctx, uint64_t* count);

/* ---- stage-level entry points (device pointers; one tensor) --------------
 * extract_mantissa_kernel (src/ANSCompressor.cpp:258-279, host :945-1009),
 * byte_histogram_kernel (:109-126, host :393-411),
 * normalize_histogram (:416-503; host arithmetic, no device involved). */
int chk_split(chk_context* ctx, const void* d_src, uint64_t num_elements, uint8_t dtype, void* d_masked,
              void* d_sidecar);
/* Inverse of chk_split: out = masked | low bytes (include/checkers/ANSCompressor.hpp:170).  The restore path does
 * this inside its decode kernel; the stand-alone stage exists for per-stage measurements. */
int chk_merge(chk_context* ctx, const void* d_masked, const void* d_sidecar, uint64_t num_elements, uint8_t dtype,
              void* d_out);
int chk_byte_histogram(chk_context* ctx, const void* d_data, uint64_t n_bytes, uint32_t hist_out[256]);
int chk_normalize_histogram(const uint32_t hist[256], int ensure_full_alphabet, int repair, uint32_t norm_freq[256],
                            uint32_t cum_freq[257], uint32_t x_max[256], uint32_t* sum_out);

/* ---- timing: the reference's [TIMING] / per-tensor ms fields -------------
 * Keys: split_hist_ms (counting), table_ms (what of the table building the counting did not hide),
 * encode_ms (lanes, offsets and gather: one kernel), compress_device_ms, encode_teams, workspace_mb,
 * d2h_ms, io_ms, compress_total_ms, h2d_ms, decode_ms, decompress_total_ms,
 * analyze_stats_ms, analyze_cluster_ms.  Device spans are CUDA-event times. */
int chk_get_timing(chk_context* ctx, const char* key, double* ms);
/* The CUDA stream (cudaStream_t) all of this context's work is issued on, so a
 * caller can order its own work or record events against it. */
int chk_get_stream(chk_context* ctx, void** stream_out);
/* Kernels launched by this context since creation. */
int chk_kernel_launches(chk_context* ctx, uint64_t* count);

/* ---- prefix-mask Re-Pair size estimator -----------------------------------
 * The reference ships this as a stand-alone, single-threaded CPU tool
 * (src/tensor_group_prefix_mask_repair.cpp).  These two calls are its compute
 * core on the GPU; `python -m checkers_b200.repair <export_dir> [...]` is the
 * command-line front end with the reference's arguments and report files.
 * Token ids: masked word >> masked_bits for tensor words, 0x80000000 + r for
 * the symbol introduced by rule r.  h_raw is HOST memory (the tool reads files):
 * numel little-endian words of storage_bytes (2 or 4) bytes.
 *
 * chk_repair_build: build_masked_sequence + build_shared_grammar (:328-352,
 *   :423-453) on the representative tensor.  Fills up to max_rules rules
 *   (lhs, rhs ids and the pair count when it was chosen), the length of the
 *   rewritten sequence, the largest pair count seen, and how many rounds had
 *   several pairs at the maximum (resolved on the host in the reference's
 *   hash-map order).
 * chk_repair_apply: build_masked_sequence + apply_existing_grammar (:455-463)
 *   on another tensor of the group; returns the rewritten length. */
const char* chk_repair_last_error(void);
int chk_repair_build(int device, const void* h_raw, uint64_t numel, uint32_t storage_bytes, uint32_t masked_bits,
                     uint32_t max_rules, uint32_t* rule_lhs, uint32_t* rule_rhs, uint64_t* rule_freq,
                     uint32_t* n_rules_out, uint64_t* tokens_out, uint64_t* max_pair_frequency_out,
                     uint64_t* tie_rounds_out);
int chk_repair_apply(int device, const void* h_raw, uint64_t numel, uint32_t storage_bytes, uint32_t masked_bits,
                     const uint32_t* rule_lhs, const uint32_t* rule_rhs, uint32_t n_rules, uint64_t* tokens_out);

/* ---- host-resident state, streamed through the GPU in chunks ---------------
 * Has no counterpart in the reference, which compresses device-resident tensors one by one under a
 * global mutex (src/ANSCompressor.cpp:1204-1280) and has no reader.
 *
 * For state that lives in host memory or does not fit into HBM (a 70B-class checkpoint in pieces of
 * about 1 GiB).  Tensors are added in order (HOST pointers; pinned memory for full copy speed) and cut
 * into consecutive parts of at most chunk_bytes.  `slots` (1..8, 3 is enough to keep the copy-in engine,
 * the SMs and the copy-out engine busy at once) device staging buffers and contexts are shared by all
 * parts, so device memory is slots x (chunk + its compress workspace) whatever the size of the state.
 * chk_stream_compress leaves every part as a complete triple of reference-format file images in pinned
 * host memory owned by the stream (chk_stream_get_image; chk_stream_save writes them as
 * <dir>/part_<k>/rank_<r>_states.ansc, mantissa/..., tables/...); chk_stream_restore decodes the parts
 * (as left by compress, or read back by chk_stream_load) into host_dst[i] for tensor i (NULL array: into
 * the tensors' own buffers; NULL entry: skip).  One call drives all parts from one host thread per slot.
 * Timing keys (sums over parts, CUDA-event times, so engines that overlap add up to more than the wall
 * time): compress_h2d_ms, compress_kernel_ms, compress_d2h_ms, compress_wall_ms, restore_h2d_ms,
 * restore_kernel_ms, restore_d2h_ms, restore_wall_ms. */
typedef struct chk_stream chk_stream;
int chk_stream_create(int device, int rank, uint64_t chunk_bytes, int slots, chk_stream** out);
/* An option of chk_set_option for every context the pipeline uses (e.g. "format_version" = 3); before the first
 * compress or load. */
int chk_stream_set_option(chk_stream* s, const char* key, int64_t value);
int chk_stream_destroy(chk_stream* s);
int chk_stream_add_tensor(chk_stream* s, const char* name, void* host_ptr, uint64_t num_elements, uint8_t dtype);
int chk_stream_compress(chk_stream* s);
int chk_stream_restore(chk_stream* s, void* const* host_dst);
int chk_stream_part_count(chk_stream* s, uint64_t* parts);
int chk_stream_part_info(chk_stream* s, uint64_t part, uint64_t* first_tensor, uint64_t* n_tensors);
int chk_stream_get_image(chk_stream* s, uint64_t part, int which, const void** data, uint64_t* size);
int chk_stream_get_summary(chk_stream* s, chk_summary* out);
int chk_stream_save(chk_stream* s, const char* output_dir);
int chk_stream_load(chk_stream* s, const char* input_dir);
int chk_stream_get_timing(chk_stream* s, const char* key, double* ms);

/* ---- encode one tensor without allocating anything -----------------------
 * Has no counterpart in the reference (which allocates and frees device
 * buffers per tensor, src/ANSCompressor.cpp:348-388).
 *
 * For callers that must not allocate when they compress: a checkpoint hook
 * running while the training step holds nearly all of HBM, a process whose
 * device memory belongs to another framework's allocator, a latency-bound loop
 * that cannot risk the allocator synchronising the device.  Every other entry
 * point of this library takes its working memory from a CUDA memory pool; this
 * one uses a fixed region compiled into the library, calls no allocation
 * routine of any kind, needs no context, and is limited to tensors of at most
 * CHK_STATIC_MAX_TENSOR_BYTES bytes (larger ones return CHK_ERR_CAPACITY).
 *
 *   d_src            device pointer, num_elements of `dtype`
 *   norm_freq/cum_freq  HOST arrays: the table to encode with (e.g. from
 *                    chk_normalize_histogram over the tensor's masked bytes)
 *   d_payload        device buffer of at least num_elements*elem_size bytes;
 *                    receives the lane streams laid out as in the .ansc data
 *                    section, or the masked tensor if the passthrough rule fires
 *   d_lane_headers   device buffer of 256*16 bytes; receives the on-disk headers
 *   payload_size_out, is_raw_out   host results
 *   stream           cudaStream_t to run on (NULL = the default stream)
 *
 * The region is per GPU and costs about 8.3 MiB of device memory on every GPU
 * the library is loaded on, for the life of the process.  All calls on one GPU
 * share it: calls that could overlap on the device must be serialised by the
 * caller (same stream, or explicit ordering).  It keeps the last call's bytes;
 * the call itself resets what has to start at zero.  The first call on each
 * device looks the region's address up (cudaGetSymbolAddress) with that device
 * current: make that first call before any stream capture begins.  The call
 * returns after the stream has drained. */
#define CHK_STATIC_MAX_TENSOR_BYTES (4u << 20)
int chk_encode_tensor_static(const void* d_src, uint64_t num_elements, uint8_t dtype, const uint32_t norm_freq[256],
                             const uint32_t cum_freq[257], void* d_payload, void* d_lane_headers,
                             uint64_t* payload_size_out, int* is_raw_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif
