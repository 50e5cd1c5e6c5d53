/*
 * checkers_oracle.h -- CPU restatement of the Checkers checkpoint-compression
 * path.  TEST INFRASTRUCTURE ONLY: this library is the checker the CUDA path is
 * compared against (tests, the smoke check and the timed CPU baseline).  The
 * shipped library never links, loads or calls it.
 *
 * Every function states which reference source range it follows (paths are
 * relative to the Checkers project root).  Parity pin: the reference has no
 * tests, golden vectors or fixtures for this path; the pins are (1) the
 * reference's own function text compiled for the CPU by oracle/build_ref.sh
 * into oracle/_ref/ and compared function-by-function in tests/test_oracle_vs_ref.py,
 * and (2) the fixtures under tests/golden/ generated from that build.
 *
 * Plain C ABI so ctypes can bind it.
 */
#ifndef CHECKERS_ORACLE_H
#define CHECKERS_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* DataType tags: include/checkers/TensorResource.hpp:30-37 */
enum { ORC_F32 = 0, ORC_BF16 = 1, ORC_F16 = 2, ORC_I8 = 3, ORC_I32 = 4, ORC_UNKNOWN = 255 };

#define ORC_LANES 256u
#define ORC_SCALE_BITS 12u
#define ORC_M 4096u
#define ORC_L (1u << 23)

/* 16-byte per-lane header: include/checkers/ANSCompressor.hpp:79-84 */
typedef struct {
    uint32_t final_state;
    uint32_t byte_count;
    uint32_t buf_offset;
    uint32_t pad;
} orc_lane_header;

/* element size / sidecar bytes per element for a dtype tag
 * (TensorResource.hpp:39-48, src/ANSCompressor.cpp:955-967). */
uint32_t orc_elem_size(int dtype);
uint32_t orc_sidecar_per_elem(int dtype);

/* src/ANSCompressor.cpp:258-279 -- masked copy + packed low bytes. */
void orc_split(const uint8_t* src, size_t n_elem, uint32_t es, uint32_t spe,
               uint8_t* masked, uint8_t* sidecar);

/* src/ANSCompressor.cpp:109-126 -- 256-bin byte histogram. */
void orc_byte_histogram(const uint8_t* data, size_t n_bytes, uint32_t hist[256]);

/* src/ANSCompressor.cpp:416-503 -- histogram -> 12-bit table.
 * Returns sum(norm_freq) (4096 for a valid model; the reference's one-pass
 * over-assignment fix can leave more). */
uint32_t orc_normalize(const uint32_t hist[256], int ensure_full_alphabet,
                       uint32_t norm_freq[256], uint32_t cum_freq[257], uint32_t x_max[256]);

/* Same, but the decrement pass repeats until the sum is 4096 (documented
 * deviation used only by the opt-in "repair tables" mode). */
uint32_t orc_normalize_repaired(const uint32_t hist[256], int ensure_full_alphabet,
                                uint32_t norm_freq[256], uint32_t cum_freq[257], uint32_t x_max[256]);

/* src/ANSCompressor.cpp:154-211 -- one lane, written backward into
 * region[0..max_chunk).  Returns byte_count; *final_state gets the state. */
uint32_t orc_encode_lane(const uint8_t* data, size_t n_bytes, uint32_t lane,
                         const uint32_t norm_freq[256], const uint32_t cum_freq[257],
                         const uint32_t x_max[256], uint8_t* region, size_t max_chunk,
                         uint32_t* final_state);

/* src/ANSCompressor.cpp:509-718 -- all 256 lanes + prefix sum + compaction +
 * passthrough rule.  `out` must hold max(2*ceil(B/256)*256, B) bytes.
 * Returns the payload size; headers[256] are the on-disk lane headers;
 * *is_raw is 1 when the passthrough rule fired. */
size_t orc_compress_tensor(const uint8_t* data, size_t n_bytes,
                           const uint32_t norm_freq[256], const uint32_t cum_freq[257],
                           const uint32_t x_max[256], orc_lane_header headers[256],
                           uint8_t* out, int* is_raw, int n_threads);

/* Decoder (absent in the reference; inverse of :154-211 using the decode
 * tables of :492-500).  Writes n_bytes to `masked_out`.  Returns 0, or a
 * negative code: -1 table sum != 4096, -2 a lane did not end in state 2^23,
 * -3 a lane did not consume exactly byte_count bytes, -4 payload too short. */
int orc_decode_tensor(const uint8_t* payload, size_t payload_size,
                      const orc_lane_header headers[256], int is_raw,
                      const uint32_t norm_freq[256], const uint32_t cum_freq[257],
                      size_t n_bytes, uint8_t* masked_out, int n_threads);

/* masked | sidecar -> original (include/checkers/ANSCompressor.hpp:170). */
void orc_merge(const uint8_t* masked, const uint8_t* sidecar, size_t n_elem,
               uint32_t es, uint32_t spe, uint8_t* out);

/* src/TensorAnalyzer.cpp:64-198 -- per-tensor statistics in float, the 256
 * thread-strided partial sums and the shared-memory tree in the same order,
 * no fused multiply-add.  hist gets min(bins,256) counters. */
void orc_tensor_stats(const void* data, size_t n_elem, int dtype, uint32_t bins,
                      uint32_t hist[256], float moments[4], float minmax[2]);

/* src/TensorAnalyzer.cpp:440-598 -- per-category union-find clustering of the
 * 5-float fingerprints.  names: n C strings.  cluster_id[i] gets -1 or the id;
 * anchor_index[c] gets the tensor index of cluster c's anchor (capacity n).
 * Returns the number of clusters. */
int orc_build_clusters(size_t n, const char* const* names, const float* fingerprints /* n*5 */,
                       int* cluster_id, int* anchor_index);

/* src/ANSCompressor.cpp:1014-1401 + writers :751-931 -- the whole
 * compress_and_save_all over host-resident tensors.
 * cluster_id[i]: -1 singleton, >=0 member, INT32_MIN = name absent from the
 * cluster map (also singleton).  anchor_names[c] for c in [0, n_clusters).
 * repair_tables != 0 selects orc_normalize_repaired for anchor tables.
 * Returns 0 on success. */
int orc_compress_and_save(size_t n, const char* const* names, const void* const* data,
                          const uint64_t* num_elements, const uint8_t* dtypes,
                          const int32_t* cluster_id, int n_clusters,
                          const char* const* anchor_names, int rank, const char* out_dir,
                          int repair_tables, int n_threads);

/* Reader + decoder for the three per-rank files.  Looks tensor `name` up in
 * <dir>/rank_<r>_states.ansc, decodes and merges its sidecar into out
 * (capacity out_cap).  Returns bytes written or a negative code
 * (-10 not found, -11 bad file, -12 capacity, else orc_decode_tensor codes). */
int64_t orc_load_tensor(const char* dir, int rank, const char* name, uint8_t* out, size_t out_cap);

/* Number of tensors in the states file, or negative on error; names are
 * copied into names_out (n_cap * 256 bytes) when non-NULL. */
int64_t orc_list_tensors(const char* dir, int rank, char* names_out, size_t n_cap);

/* Timed CPU baseline: the whole hot path over n host tensors with `n_threads`
 * OpenMP threads, one tensor per thread at a time (split, histogram, table,
 * 256 lanes, compaction; then decode and merge, checked against the input).
 * seconds_out[0] = compress, [1] = decompress; bytes_out[0] = original bytes,
 * [1] = payload bytes, [2] = sidecar bytes.  Returns 0, or -1 if a round trip
 * did not reproduce its input. */
int orc_roundtrip_timed(size_t n, const void* const* data, const uint64_t* num_elements, const uint8_t* dtypes,
                        int n_threads, double seconds_out[2], uint64_t bytes_out[3]);

#ifdef __cplusplus
}
#endif
#endif
