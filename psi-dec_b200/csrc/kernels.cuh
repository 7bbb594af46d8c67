// Launch interface between the C ABI (api.cu) and the sm_100a kernels.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "host_logic.hpp"

namespace psi {

// Device scalar block rewritten by every prepare (the analogue of the reference's replay parameter buffer).
enum ScalarSlot : uint32_t {
    kScalarNumActiveTokens = 0,
    kScalarNumCtas = 1,
    kScalarNumReduces = 2,
    kScalarNumChunkCtas = 3,
    kScalarCount = 8
};

struct PageGeometry {
    const void* pages;
    const uint32_t* page_ids;     // whole table
    uint64_t page_elems;          // elements per page
    uint64_t num_pages;           // pages of the arena (bounds of the TMA view; 0 where no kernel needs it)
    uint32_t layer;
    uint32_t num_layers;
    uint32_t pages_per_req;       // num_blocks * num_page_ids_per_block: one (slot, layer) row of the table
    uint32_t tokens_per_page;
    uint32_t num_kv_heads;
    uint32_t head_dim;
    uint32_t elem_bytes;
    uint32_t* fault;              // nullptr, or the status word a failed bounds check writes PSI_ERR_PAGE_ID to
};

struct AppendParams {
    PageGeometry geo;
    const void* flat_k;
    const void* flat_v;
    const uint32_t* req_slots;
    const uint32_t* flat_token_indices;
    const uint32_t* scalars;
    uint32_t num_total_tokens;    // launch capacity; rows >= scalars[kScalarNumActiveTokens] do nothing
};

struct PrepParams {
    PageGeometry geo;
    const void* q_in;             // [T][Hq][D] projected, not yet normalised
    const void* k_in;             // [T][Hkv][D]
    const void* v_in;             // [T][Hkv][D]
    void* q_out;                  // [T][Hq][D] normalised + rotated
    const void* q_weight;         // bf16 [D]
    const void* k_weight;         // bf16 [D]
    const float* inverse_frequencies;  // [rope_dim / 2]
    float attention_factor;
    float eps;
    uint32_t rope_dim;
    uint32_t num_q_heads;
    uint32_t dtype;
    const uint32_t* req_slots;
    const uint32_t* flat_token_indices;
    const uint32_t* scalars;
    uint32_t num_total_tokens;
    // Source strides in elements: row (token, head) of q starts at token * q_token_stride + head * q_head_stride, of
    // k / v at token * kv_token_stride + head * head_dim.  Contiguous [T][H][D] inputs and the rows of a fused
    // projection output [T][q|g pairs, k heads, v heads] are both described this way.
    uint64_t q_token_stride;
    uint64_t q_head_stride;
    uint64_t kv_token_stride;
    const void* g_in;             // gate rows, strided like q_in; nullptr without gates
    void* g_out;                  // [T][Hq][D] contiguous copy of the gate rows
};

struct GatherParams {
    PageGeometry geo;
    uint32_t req_slot;
    uint32_t tok_begin;
    uint32_t tok_end;
    void* k_out;
    void* v_out;
};

// KV-range exchange fused into the map launch: every rank of a group holds one slice of each sequence's KV range and
// writes its partial (o, m, l) into its slot of the owner's receive area (peer-mapped memory, plain stores).  The CTA
// that finishes a rank's launch last publishes the rank's arrival flag; on the owner the CTAs then wait, with a bound,
// for every rank's flag and merge the partials into `out`.  `flag == nullptr` means the launch has no exchange.
struct ExchangeParams {
    uint32_t* flag;               // this rank's arrival flag, in the owner's memory as mapped on this device
    const uint32_t* consumed;     // the owner's "last merged step" word, as mapped on this device
    uint32_t* sync_words;         // this device, zero between launches: [0] launch arrivals, [1] merge arrivals, [2] verdict
    const float* recv;            // owner only: this step's receive area in local memory, `world` slots of `slot_stride`
    const uint32_t* flags;        // owner only: the `world` arrival flags, local memory
    uint32_t* consumed_local;     // owner only: the consumed word, local memory
    uint64_t slot_stride;         // floats from one rank's slot to the next; a slot is o [rows][D] | m [rows] | l [rows]
    uint32_t world;
    uint32_t step;                // 1, 2, 3, ...: flag value of this step; slot parity = step & 1
    uint32_t max_polls;           // bound of every wait (about 100 ns per poll)
    uint32_t num_rows;            // query tokens * q heads
};

enum SyncWord : uint32_t { kSyncLaunchArrivals = 0, kSyncMergeArrivals = 1, kSyncVerdict = 2, kSyncWordCount = 4 };

struct AttendParams {
    PageGeometry geo;
    const void* q;
    void* out;                    // [T][Hq][D] in the I/O dtype, or nullptr when ext_* are set
    float* ext_o;                 // [T][Hq][D] f32 normalised partial (attend_partial), else nullptr
    float* ext_m;                 // [T][Hq] natural-log max
    float* ext_l;                 // [T][Hq] exp-sum
    const void* gates;            // nullptr, or [T][Hq][D] in the I/O dtype: out = attention * sigmoid(gate)
    const void* new_k;            // fused step only: this step's K rows [T][Hkv][D], appended by the map kernel
    const void* new_v;            //                  and read from here instead of from their pages; else nullptr
    const DeviceItem* items;
    const uint32_t* cta_item_begin;
    const DeviceItem* cta_first_items;  // nullptr, or [num_ctas]: a copy of each CTA's first item, readable before its range
    const ReduceUnit* reduces;
    float* partial_o;             // [slots][16][D] normalised
    float* partial_m;             // [slots][16] log2-domain max
    float* partial_l;             // [slots][16]
    uint32_t* unit_counters;      // [reduce units], zero between launches: arrivals of a unit's items (mma kernel)
    const uint32_t* scalars;
    uint32_t num_q_heads;
    uint32_t tokens_per_tile;     // query tokens of one 16-row tile (plan geometry)
    uint32_t dtype;
    float scale_log2;             // scale * log2(e)
    uint32_t* status;             // nullptr, or the word a bounded device-side wait writes PSI_ERR_TIMEOUT to
    uint32_t tma_feed;            // decode kernel: whole K/V tiles by TMA boxes instead of cp.async (PSI_KERNEL_MMA_TMA)
    ExchangeParams xchg;          // KV-range exchange in the same launch (mma kernel); xchg.flag == nullptr: none
};

struct CombineParams {
    const float* const* o;        // device array of n pointers
    const float* const* m;
    const float* const* l;
    const uint32_t* flags;        // nullptr, or n arrival flags in this device's memory: wait until each >= flag_value
    uint32_t flag_value;
    uint32_t max_polls;           // bound of the wait; on expiry *status = PSI_ERR_TIMEOUT and nothing is written
    uint32_t* status;
    uint32_t* sync_words;         // with flags: this device's sync words (zero between launches), see SyncWord
    uint32_t n;
    uint32_t num_rows;            // num_tokens * Hq
    uint32_t head_dim;
    uint32_t dtype;
    void* out;
};

// Dense bidirectional block attention partials (one warp per (token, q head)).
struct BlockPartialParams {
    const void* q;                 // [T][Hq][D]
    const void* local_k;           // [T][Hkv][D]
    const void* local_v;           // [T][Hkv][D]
    const uint32_t* slot_indices;  // nullptr (slot = token) or [T]: partial slot of each token
    float* o;                      // [slots][Hq][D] normalised
    float* m;                      // [slots][Hq] natural-log max
    float* l;                      // [slots][Hq] exp-sum
    uint32_t num_tokens;
    uint32_t block_size;
    uint32_t num_q_heads;
    uint32_t num_kv_heads;
    uint32_t head_dim;
    uint32_t dtype;
    float scale;
};
cudaError_t launch_block_partial(const BlockPartialParams& p, cudaStream_t stream);

cudaError_t launch_kv_append(const AppendParams& p, cudaStream_t stream);
cudaError_t launch_page_gather(const GatherParams& p, cudaStream_t stream);
// One launch that copies three host-mapped (pinned) buffers into device memory; sizes are multiples of 16 bytes.
constexpr int kPullBuffers = 4;
cudaError_t launch_host_pull(const void* const src[kPullBuffers], void* const dst[kPullBuffers],
                             const uint64_t bytes[kPullBuffers], cudaStream_t stream);
cudaError_t launch_norm_rope_append(const PrepParams& p, cudaStream_t stream);

// Map kernels.  `num_ctas` CTAs walk cta_item_begin.  The generic kernel takes any profile with head_dim <= 256; the
// mma kernel needs bf16/f16, head_dim in {64,128,256} and tokens_per_page % 8 == 0.
bool attend_mma_supported(uint32_t dtype, uint32_t head_dim, uint32_t tokens_per_page);
uint32_t attend_mma_ctas_per_sm(uint32_t head_dim);
// Resident CTAs per SM of the CUDA-core map kernel that a profile of this head_dim and dtype gets (the staged kernel
// when head_dim is a multiple of four, else the one-warp kernel).
uint32_t attend_generic_ctas_per_sm(uint32_t head_dim, uint32_t dtype);
uint32_t attend_staged_ctas_per_sm(uint32_t dtype);
// The staged CUDA-core map kernel (attend_staged.cu): taken by launch_attend_generic when the launch qualifies.
bool attend_staged_supported(const AttendParams& p);
cudaError_t launch_attend_staged(const AttendParams& p, uint32_t num_ctas, cudaStream_t stream);
cudaError_t launch_attend_generic(const AttendParams& p, uint32_t num_ctas, cudaStream_t stream);
cudaError_t launch_attend_mma(const AttendParams& p, uint32_t num_ctas, cudaStream_t stream);
// Long query runs: one CTA = up to eight query tiles of one request sharing one pass over the KV range.
bool attend_chunk_supported(uint32_t dtype, uint32_t head_dim, uint32_t tokens_per_page);
cudaError_t launch_attend_chunk(const AttendParams& p, uint32_t num_ctas, cudaStream_t stream);
// The same work items on the tcgen05 tensor cores (accumulators in TMEM); same profiles as launch_attend_chunk.
// Streams `bytes` of device memory through 16-byte read-only loads (bandwidth probe; writes nothing but one sink word).
cudaError_t launch_read_stream(const void* src, uint64_t bytes, uint32_t* sink, uint32_t num_ctas, cudaStream_t stream);

cudaError_t launch_attend_chunk_umma(const AttendParams& p, uint32_t num_ctas, cudaStream_t stream);
cudaError_t launch_attend_reduce(const AttendParams& p, uint32_t num_reduces, cudaStream_t stream);
cudaError_t launch_combine(const CombineParams& p, cudaStream_t stream);
// KV-range exchange without the fused attention launch: push a finished local partial into the rank's slot and publish
// the flag; on the owner, wait for every rank and merge (at most `max_ctas` CTAs, one row each at a time).
cudaError_t launch_exchange_push(const ExchangeParams& x, const float* local, float* slot, uint64_t floats,
                                 uint32_t* status, cudaStream_t stream);
cudaError_t launch_exchange_merge(const ExchangeParams& x, void* out, uint32_t dtype, uint32_t head_dim, uint32_t* status,
                                  uint32_t max_ctas, cudaStream_t stream);
// Release-stores `value` to *flag (local or peer memory) once all earlier work of the stream is visible system-wide.
cudaError_t launch_signal(uint32_t* flag, uint32_t value, cudaStream_t stream);

}  // namespace psi
