/*
 * CPU oracle for the paged GQA decode path of psi-dec.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the reference's algorithms for the path:
 * KV page write (append), page gather, projected GQA attention with exact
 * softmax, the split-KV partial merge, the batch-metadata / KV-split planner,
 * the replay bucket policy, the SplitKV variant selector and the page-ID
 * allocator.  Each function cites the reference file:line it follows (paths
 * are relative to the reference project root).
 *
 * It is the checker: only the test-suite, the smoke entry and the benchmark's
 * cpu_baseline / reference arm may load it.  The CUDA library never links,
 * loads or calls anything here.
 *
 * Pinning: the reference is Rust + Metal and cannot be compiled or run where
 * this oracle is built, so the oracle is pinned against the known-answer and
 * golden vectors that the reference's own tests hold for the path (closed-form
 * causal attention, KV write bytes, metadata vectors, bucket vectors, variant
 * matrix, allocator bitmaps); tests/test_oracle_golden.py holds them.
 * bf16 rounding (crate `half` 2.7, round-to-nearest-even) is restated here
 * and is "parity unpinned" at that one boundary: the reference's tests never
 * pin `half` itself.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>
#include <unistd.h>

#define PSI_ORACLE_API __attribute__((visibility("default")))

enum { PSI_O_F32 = 0, PSI_O_BF16 = 1, PSI_O_F16 = 2 };

/* ------------------------------------------------------------------ */
/* dtype conversion                                                    */
/* ------------------------------------------------------------------ */

static inline uint32_t f32_bits(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
}

static inline float bits_f32(uint32_t u) {
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* IEEE round-to-nearest-even f32 -> bf16, quiet NaN preserved (crate `half` bf16::from_f32). */
PSI_ORACLE_API uint16_t psi_oracle_f32_to_bf16(float f) {
    uint32_t u = f32_bits(f);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) {
        return (uint16_t)((u >> 16) | 0x0040u);
    }
    uint32_t round_bit = 0x00008000u;
    if ((u & round_bit) != 0 && (u & (3u * round_bit - 1u)) != 0) {
        return (uint16_t)((u >> 16) + 1u);
    }
    return (uint16_t)(u >> 16);
}

PSI_ORACLE_API float psi_oracle_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

PSI_ORACLE_API float psi_oracle_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    if (exp == 0) {
        if (man == 0) return bits_f32(sign);
        /* subnormal: normalise */
        int e = -1;
        do {
            man <<= 1;
            ++e;
        } while ((man & 0x400u) == 0);
        man &= 0x3FFu;
        return bits_f32(sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13));
    }
    if (exp == 31) return bits_f32(sign | 0x7F800000u | (man << 13));
    return bits_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

/* IEEE round-to-nearest-even f32 -> f16. */
PSI_ORACLE_API uint16_t psi_oracle_f32_to_f16(float f) {
    uint32_t u = f32_bits(f);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t abs = u & 0x7FFFFFFFu;
    if (abs > 0x7F800000u) return (uint16_t)(sign | 0x7E00u);
    if (abs >= 0x47800000u) return (uint16_t)(sign | 0x7C00u); /* overflow -> inf (65520 rounds up) */
    if (abs >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);
    if (abs < 0x33000001u) return (uint16_t)sign; /* below half of the smallest subnormal */
    int32_t exp = (int32_t)(abs >> 23) - 127;
    uint32_t man = (abs & 0x7FFFFFu) | 0x800000u;
    uint32_t shift;
    uint32_t half_exp;
    if (exp < -14) {
        shift = (uint32_t)(13 + (-14 - exp));
        half_exp = 0;
    } else {
        shift = 13;
        half_exp = (uint32_t)(exp + 15);
    }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) ++q;
    uint32_t out;
    if (half_exp == 0) {
        out = q; /* may carry into exponent 1: correct */
    } else {
        out = ((half_exp - 1u) << 10) + q; /* q holds the hidden bit: adds one to the exponent */
    }
    return (uint16_t)(sign | out);
}

static inline size_t dtype_size(int dtype) { return dtype == PSI_O_F32 ? 4 : 2; }

static inline float load_elem(const void* base, size_t index, int dtype) {
    if (dtype == PSI_O_F32) return ((const float*)base)[index];
    uint16_t h = ((const uint16_t*)base)[index];
    return dtype == PSI_O_BF16 ? psi_oracle_bf16_to_f32(h) : psi_oracle_f16_to_f32(h);
}

PSI_ORACLE_API void psi_oracle_decode(const void* src, int dtype, size_t n, float* dst) {
    for (size_t i = 0; i < n; ++i) dst[i] = load_elem(src, i, dtype);
}

PSI_ORACLE_API void psi_oracle_encode(const float* src, int dtype, size_t n, void* dst) {
    for (size_t i = 0; i < n; ++i) {
        if (dtype == PSI_O_F32) {
            ((float*)dst)[i] = src[i];
        } else if (dtype == PSI_O_BF16) {
            ((uint16_t*)dst)[i] = psi_oracle_f32_to_bf16(src[i]);
        } else {
            ((uint16_t*)dst)[i] = psi_oracle_f32_to_f16(src[i]);
        }
    }
}

/* ------------------------------------------------------------------ */
/* Page addressing                                                     */
/* ------------------------------------------------------------------ */

typedef struct {
    uint32_t num_req_slots;
    uint32_t num_gqa_layers;
    uint32_t num_blocks;
    uint32_t num_page_ids_per_block;
} psi_oracle_layout;

/* Table index of the page that holds `token_index`.
 * crates/inference-backend-metal/src/components/metal/gqa_kv_page_write.metal:29-37 */
static inline uint64_t table_index(const psi_oracle_layout* L, uint32_t req_slot, uint32_t layer, uint32_t token_index,
                                   uint32_t tokens_per_page) {
    uint32_t block_index = token_index / (tokens_per_page * L->num_page_ids_per_block);
    uint32_t page_id_index = (token_index / tokens_per_page) % L->num_page_ids_per_block;
    return ((((uint64_t)req_slot * L->num_gqa_layers + layer) * L->num_blocks + block_index) *
            L->num_page_ids_per_block) +
           page_id_index;
}

/* KV append.  Pure bit copy of element size `elem_bytes` (2 or 4).
 * crates/inference-backend-metal/src/components/metal/gqa_kv_page_write.metal:6-53 */
PSI_ORACLE_API void psi_oracle_kv_page_write(void* pages, uint32_t elem_bytes, const void* flat_k, const void* flat_v,
                                             const uint32_t* req_slots, const uint32_t* flat_token_indices,
                                             const uint32_t* page_ids, uint32_t num_active_token_writes,
                                             uint32_t layer, const psi_oracle_layout* L, uint32_t num_kv_heads,
                                             uint32_t head_dim, uint32_t page_bytes) {
    uint32_t tokens_per_page = page_bytes / (2u * num_kv_heads * head_dim * elem_bytes);
    uint64_t page_elems = (uint64_t)page_bytes / elem_bytes;
    uint64_t v_region = (uint64_t)num_kv_heads * tokens_per_page * head_dim;
    unsigned char* out = (unsigned char*)pages;
    const unsigned char* k = (const unsigned char*)flat_k;
    const unsigned char* v = (const unsigned char*)flat_v;
    for (uint32_t w = 0; w < num_active_token_writes; ++w) {
        uint32_t tok = flat_token_indices[w];
        uint64_t page_id = page_ids[table_index(L, req_slots[w], layer, tok, tokens_per_page)];
        uint32_t page_token = tok % tokens_per_page;
        for (uint32_t h = 0; h < num_kv_heads; ++h) {
            for (uint32_t d = 0; d < head_dim; ++d) {
                uint64_t in_page = ((uint64_t)h * tokens_per_page + page_token) * head_dim + d;
                uint64_t flat = ((uint64_t)w * num_kv_heads + h) * head_dim + d;
                memcpy(out + (page_id * page_elems + in_page) * elem_bytes, k + flat * elem_bytes, elem_bytes);
                memcpy(out + (page_id * page_elems + v_region + in_page) * elem_bytes, v + flat * elem_bytes,
                       elem_bytes);
            }
        }
    }
}

/* Page gather: the read-side of the same address algebra; tokens [tok_begin, tok_end) of one request slot into
 * contiguous [n][Hkv][D] K and V.  The reference resolves this inline in its map kernels:
 * crates/inference-backend-metal/src/components/metal/gqa_split_kv_single_q_map.metal:96-111,195-209 */
PSI_ORACLE_API void psi_oracle_page_gather(const void* pages, uint32_t elem_bytes, const uint32_t* page_ids,
                                           uint32_t req_slot, uint32_t layer, const psi_oracle_layout* L,
                                           uint32_t num_kv_heads, uint32_t head_dim, uint32_t page_bytes,
                                           uint32_t tok_begin, uint32_t tok_end, void* k_out, void* v_out) {
    uint32_t tokens_per_page = page_bytes / (2u * num_kv_heads * head_dim * elem_bytes);
    uint64_t page_elems = (uint64_t)page_bytes / elem_bytes;
    uint64_t v_region = (uint64_t)num_kv_heads * tokens_per_page * head_dim;
    const unsigned char* in = (const unsigned char*)pages;
    unsigned char* k = (unsigned char*)k_out;
    unsigned char* v = (unsigned char*)v_out;
    size_t row_bytes = (size_t)head_dim * elem_bytes;
    for (uint32_t tok = tok_begin; tok < tok_end; ++tok) {
        uint64_t page_id = page_ids[table_index(L, req_slot, layer, tok, tokens_per_page)];
        uint32_t page_token = tok % tokens_per_page;
        for (uint32_t h = 0; h < num_kv_heads; ++h) {
            uint64_t in_page = ((uint64_t)h * tokens_per_page + page_token) * head_dim;
            uint64_t flat = ((uint64_t)(tok - tok_begin) * num_kv_heads + h) * head_dim;
            memcpy(k + flat * elem_bytes, in + (page_id * page_elems + in_page) * elem_bytes, row_bytes);
            memcpy(v + flat * elem_bytes, in + (page_id * page_elems + v_region + in_page) * elem_bytes, row_bytes);
        }
    }
}

/* ------------------------------------------------------------------ */
/* Attention                                                           */
/* ------------------------------------------------------------------ */

/* crates/inference-executor-core/src/reference.rs:15-31.  Returns 0 on success, 1 when the total is not a finite
 * positive number (the reference asserts). */
PSI_ORACLE_API int psi_oracle_softmax(const float* logits, size_t n, float* out) {
    if (n == 0) return 1;
    float max_logit = -INFINITY;
    for (size_t i = 0; i < n; ++i) max_logit = logits[i] > max_logit ? logits[i] : max_logit;
    float total = 0.0f;
    for (size_t i = 0; i < n; ++i) {
        out[i] = expf(logits[i] - max_logit);
        total += out[i];
    }
    if (!(total > 0.0f) || !isfinite(total)) return 1;
    for (size_t i = 0; i < n; ++i) out[i] = out[i] / total;
    return 0;
}

/* Already-projected GQA attention over contiguous per-request K/V, f32 throughout.
 * crates/inference-executor-core/src/attn/gqa/reference.rs:15-78 (loop structure, head mapping, visibility). */
PSI_ORACLE_API int psi_oracle_projected_gqa_reference(uint32_t num_q_heads, uint32_t num_kv_heads, uint32_t head_dim,
                                                      float scale, const uint32_t* cu_tokens,
                                                      const uint32_t* token_indices, uint32_t num_reqs, const float* q,
                                                      const float* const* context_k_by_req,
                                                      const float* const* context_v_by_req, float* output) {
    uint32_t heads_per_kv_head = num_q_heads / num_kv_heads;
    int status = 0;
    for (uint32_t req = 0; req < num_reqs; ++req) {
        uint32_t req_start = cu_tokens[req];
        uint32_t req_end = cu_tokens[req + 1];
        const float* ck = context_k_by_req[req];
        const float* cv = context_v_by_req[req];
        for (uint32_t tir = 0; tir < req_end - req_start; ++tir) {
            uint32_t token = req_start + tir;
            size_t visible = (size_t)token_indices[req] + tir + 1;
            float* logits = (float*)malloc(visible * sizeof(float));
            float* prob = (float*)malloc(visible * sizeof(float));
            for (uint32_t qh = 0; qh < num_q_heads; ++qh) {
                uint32_t kvh = qh / heads_per_kv_head;
                const float* qrow = q + ((size_t)token * num_q_heads + qh) * head_dim;
                for (size_t c = 0; c < visible; ++c) {
                    const float* krow = ck + (c * num_kv_heads + kvh) * head_dim;
                    float dot = 0.0f;
                    for (uint32_t d = 0; d < head_dim; ++d) dot += qrow[d] * krow[d];
                    logits[c] = dot * scale;
                }
                status |= psi_oracle_softmax(logits, visible, prob);
                float* orow = output + ((size_t)token * num_q_heads + qh) * head_dim;
                for (uint32_t d = 0; d < head_dim; ++d) {
                    float weighted = 0.0f;
                    for (size_t c = 0; c < visible; ++c) weighted += prob[c] * cv[(c * num_kv_heads + kvh) * head_dim + d];
                    orow[d] = weighted;
                }
            }
            free(logits);
            free(prob);
        }
    }
    return status;
}

/* The same attention, reading K/V straight from the paged arena through the page table (gather fused, as in
 * gqa_split_kv_single_q_map.metal:96-111) with inputs decoded to f32 and f32 arithmetic in the reference's
 * summation order.  Output f32 [T][Hq][D].  Parallel over (flat token, q head) rows on a pthread pool; `kv_begin/kv_end`
 * (both 0 -> full range) restrict the visible range for split-KV partial checks.  Optional `out_max`/`out_sum`
 * ([T][Hq]) receive the natural-log-domain running max and exp-sum of each row.
 * Semantics: reference.rs:41-47 (token i of a request sees keys [0, token_index+i]). */
typedef struct {
    const void* pages;
    int dtype;
    const void* q;
    const uint32_t* req_slots;
    const uint32_t* flat_token_indices;
    uint32_t num_tokens;
    const uint32_t* page_ids;
    uint32_t layer;
    const psi_oracle_layout* L;
    uint32_t num_q_heads, num_kv_heads, head_dim, page_bytes;
    float scale;
    uint32_t kv_begin, kv_end;
    float* output;
    float* out_max;
    float* out_sum;
    int64_t next_row; /* shared work counter */
    int status;
} paged_job;

static void paged_attention_row(paged_job* J, int64_t row, int* status) {
    size_t esz = dtype_size(J->dtype);
    uint32_t num_q_heads = J->num_q_heads, num_kv_heads = J->num_kv_heads, head_dim = J->head_dim;
    uint32_t tokens_per_page = J->page_bytes / (2u * num_kv_heads * head_dim * (uint32_t)esz);
    uint64_t page_elems = (uint64_t)J->page_bytes / esz;
    uint64_t v_region = (uint64_t)num_kv_heads * tokens_per_page * head_dim;
    uint32_t token = (uint32_t)(row / num_q_heads);
    uint32_t qh = (uint32_t)(row % num_q_heads);
    uint32_t kvh = qh / (num_q_heads / num_kv_heads);
    uint32_t lo = 0;
    uint32_t hi = J->flat_token_indices[token] + 1;
    if (J->kv_end != 0) {
        lo = J->kv_begin;
        hi = hi < J->kv_end ? hi : J->kv_end;
    }
    float* orow = J->output + ((size_t)token * num_q_heads + qh) * head_dim;
    if (hi <= lo) {
        for (uint32_t d = 0; d < head_dim; ++d) orow[d] = 0.0f;
        if (J->out_max) J->out_max[row] = -INFINITY;
        if (J->out_sum) J->out_sum[row] = 0.0f;
        return;
    }
    size_t visible = hi - lo;
    float* qrow = (float*)malloc(head_dim * sizeof(float));
    float* logits = (float*)malloc(visible * sizeof(float));
    float* krow = (float*)malloc(head_dim * sizeof(float));
    for (uint32_t d = 0; d < head_dim; ++d)
        qrow[d] = load_elem(J->q, ((size_t)token * num_q_heads + qh) * head_dim + d, J->dtype);
    for (uint32_t c = lo; c < hi; ++c) {
        uint64_t page_id = J->page_ids[table_index(J->L, J->req_slots[token], J->layer, c, tokens_per_page)];
        uint64_t base = page_id * page_elems + ((uint64_t)kvh * tokens_per_page + c % tokens_per_page) * head_dim;
        float dot = 0.0f;
        for (uint32_t d = 0; d < head_dim; ++d) krow[d] = load_elem(J->pages, base + d, J->dtype);
        for (uint32_t d = 0; d < head_dim; ++d) dot += qrow[d] * krow[d];
        logits[c - lo] = dot * J->scale;
    }
    float max_logit = -INFINITY;
    for (size_t i = 0; i < visible; ++i) max_logit = logits[i] > max_logit ? logits[i] : max_logit;
    float total = 0.0f;
    for (size_t i = 0; i < visible; ++i) {
        logits[i] = expf(logits[i] - max_logit);
        total += logits[i];
    }
    if (!(total > 0.0f) || !isfinite(total)) *status |= 1;
    if (J->out_max) J->out_max[row] = max_logit;
    if (J->out_sum) J->out_sum[row] = total;
    for (size_t i = 0; i < visible; ++i) logits[i] = logits[i] / total;
    for (uint32_t d = 0; d < head_dim; ++d) orow[d] = 0.0f;
    /* token-outer accumulation: each orow[d] still sums its terms in increasing token order, which is the
     * reference's order per output element (reference.rs:58-66). */
    for (uint32_t c = lo; c < hi; ++c) {
        uint64_t page_id = J->page_ids[table_index(J->L, J->req_slots[token], J->layer, c, tokens_per_page)];
        uint64_t base =
            page_id * page_elems + v_region + ((uint64_t)kvh * tokens_per_page + c % tokens_per_page) * head_dim;
        float p = logits[c - lo];
        for (uint32_t d = 0; d < head_dim; ++d) orow[d] += p * load_elem(J->pages, base + d, J->dtype);
    }
    free(qrow);
    free(logits);
    free(krow);
}

static void* paged_worker(void* arg) {
    paged_job* J = (paged_job*)arg;
    int64_t total_rows = (int64_t)J->num_tokens * J->num_q_heads;
    int status = 0;
    for (;;) {
        int64_t row = __atomic_fetch_add(&J->next_row, 1, __ATOMIC_RELAXED);
        if (row >= total_rows) break;
        paged_attention_row(J, row, &status);
    }
    if (status) __atomic_fetch_or(&J->status, status, __ATOMIC_RELAXED);
    return NULL;
}

static int g_num_threads = 0;

/* Worker threads used by psi_oracle_paged_attention: 0 selects the online core count. */
PSI_ORACLE_API void psi_oracle_set_num_threads(int n) { g_num_threads = n; }

PSI_ORACLE_API int psi_oracle_num_threads(void) {
    if (g_num_threads > 0) return g_num_threads;
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}

PSI_ORACLE_API int psi_oracle_paged_attention(const void* pages, int dtype, const void* q, const uint32_t* req_slots,
                                              const uint32_t* flat_token_indices, uint32_t num_tokens,
                                              const uint32_t* page_ids, uint32_t layer, const psi_oracle_layout* L,
                                              uint32_t num_q_heads, uint32_t num_kv_heads, uint32_t head_dim,
                                              uint32_t page_bytes, float scale, uint32_t kv_begin, uint32_t kv_end,
                                              float* output, float* out_max, float* out_sum) {
    paged_job J = {pages, dtype, q, req_slots, flat_token_indices, num_tokens, page_ids, layer, L, num_q_heads,
                   num_kv_heads, head_dim, page_bytes, scale, kv_begin, kv_end, output, out_max, out_sum, 0, 0};
    int64_t total_rows = (int64_t)num_tokens * num_q_heads;
    int nthreads = psi_oracle_num_threads();
    if (nthreads > total_rows) nthreads = (int)total_rows;
    if (nthreads <= 1) {
        paged_worker(&J);
        return J.status;
    }
    pthread_t* threads = (pthread_t*)malloc(sizeof(pthread_t) * (size_t)nthreads);
    int started = 0;
    for (int i = 0; i < nthreads - 1; ++i) {
        if (pthread_create(&threads[started], NULL, paged_worker, &J) == 0) ++started;
    }
    paged_worker(&J);
    for (int i = 0; i < started; ++i) pthread_join(threads[i], NULL);
    free(threads);
    return J.status;
}

/* Split-KV partial merge for one output row.
 * crates/inference-backend-metal/src/components/metal/gqa_split_kv_single_q_reduce.metal:27-48 */
PSI_ORACLE_API void psi_oracle_merge_partials(const float* partial_output /* [n][D] normalised */,
                                              const float* partial_max, const float* partial_sum, uint32_t n,
                                              uint32_t head_dim, float* out) {
    float global_max = -INFINITY;
    for (uint32_t i = 0; i < n; ++i) global_max = partial_max[i] > global_max ? partial_max[i] : global_max;
    for (uint32_t d = 0; d < head_dim; ++d) {
        float global_sum = 0.0f;
        float acc = 0.0f;
        for (uint32_t i = 0; i < n; ++i) {
            float w = isfinite(partial_max[i]) ? expf(partial_max[i] - global_max) * partial_sum[i] : 0.0f;
            global_sum += w;
            acc += w * partial_output[(size_t)i * head_dim + d];
        }
        out[d] = global_sum > 0.0f ? acc / global_sum : 0.0f;
    }
}

/* ------------------------------------------------------------------ */
/* Replay bucket policy                                                */
/* ------------------------------------------------------------------ */

static int cmp_u32(const void* a, const void* b) {
    uint32_t x = *(const uint32_t*)a, y = *(const uint32_t*)b;
    return x < y ? -1 : (x > y ? 1 : 0);
}

/* crates/inference-executor-core/src/replay.rs:25-44,69-90.  Writes the strictly increasing bucket list into `out`
 * (capacity `out_cap`) and returns its length, or -1 on a contract violation / overflow of out_cap. */
PSI_ORACLE_API int64_t psi_oracle_bucket_policy(uint32_t max_capacity, const uint32_t* boundaries,
                                                uint32_t num_boundaries, uint32_t* out, uint64_t out_cap) {
    static const uint32_t base[14] = {1, 2, 4, 6, 8, 12, 16, 20, 24, 32, 40, 48, 56, 64};
    if (max_capacity == 0) return -1;
    uint64_t n = 0;
#define PUSH(v)                         \
    do {                                \
        if (n >= out_cap) return -1;    \
        out[n++] = (v);                 \
    } while (0)
    for (int i = 0; i < 14 && base[i] <= max_capacity; ++i) PUSH(base[i]);
    uint32_t lower = 64;
    int done = 0;
    while (!done && lower < max_capacity) {
        uint32_t step = lower / 4;
        for (uint32_t part = 1; part <= 4; ++part) {
            uint64_t cand64 = (uint64_t)lower + (uint64_t)step * part;
            uint32_t cand = cand64 > UINT32_MAX ? UINT32_MAX : (uint32_t)cand64;
            if (cand >= max_capacity) {
                done = 1;
                break;
            }
            PUSH(cand);
        }
        uint64_t next = (uint64_t)lower * 2;
        lower = next > UINT32_MAX ? UINT32_MAX : (uint32_t)next;
    }
    for (uint32_t i = 0; i < num_boundaries; ++i) {
        uint32_t b = boundaries[i];
        if (b == 0) return -1;
        if (b > 1 && b <= max_capacity) PUSH(b - 1);
    }
    PUSH(max_capacity);
#undef PUSH
    qsort(out, n, sizeof(uint32_t), cmp_u32);
    uint64_t m = 0;
    for (uint64_t i = 0; i < n; ++i)
        if (m == 0 || out[m - 1] != out[i]) out[m++] = out[i];
    return (int64_t)m;
}

/* replay.rs:57-62: first bucket >= active.  Returns 0 on a contract violation. */
PSI_ORACLE_API uint32_t psi_oracle_bucket_capacity(const uint32_t* buckets, uint64_t n, uint32_t active) {
    if (active == 0 || n == 0 || active > buckets[n - 1]) return 0;
    uint64_t lo = 0, hi = n;
    while (lo < hi) {
        uint64_t mid = (lo + hi) / 2;
        if (buckets[mid] < active) lo = mid + 1; else hi = mid;
    }
    return buckets[lo];
}

/* ------------------------------------------------------------------ */
/* SplitKV variant selector                                            */
/* ------------------------------------------------------------------ */

typedef struct {
    uint32_t tiled_q;            /* 0 = SingleQ, 1 = TiledQ */
    uint32_t q_token_tile_size;  /* TiledQ only, else 0 */
    uint32_t kv_token_tile_size;
    uint32_t num_threads_per_threadblock; /* SingleQ only, else 0 */
    uint32_t q_head_tile_size;
} psi_oracle_variant;

static uint32_t next_pow2_u32(uint32_t v) {
    uint32_t p = 1;
    while (p < v) p <<= 1;
    return p;
}

/* crates/inference-backend-metal/src/components/gqa_split_kv.rs:85-157.  `dspark_history` selects the SingleQ-only
 * profile of new_dspark_history.  Returns 0 on success, 1 on invalid config. */
PSI_ORACLE_API int psi_oracle_split_kv_select(int io_dtype, uint32_t page_bytes, uint32_t num_q_heads,
                                              uint32_t num_kv_heads, uint32_t head_dim, int dspark_history,
                                              uint32_t num_tokens, uint32_t num_q_token_tiles,
                                              psi_oracle_variant* out, uint32_t* max_q_tokens_per_partial) {
    if (!(io_dtype == PSI_O_F32 || io_dtype == PSI_O_BF16)) return 1;
    if (page_bytes == 0 || num_q_heads == 0 || num_kv_heads == 0 || head_dim == 0) return 1;
    if (num_q_heads % num_kv_heads != 0) return 1;
    uint64_t per_token = (uint64_t)num_kv_heads * head_dim * 2u * (io_dtype == PSI_O_F32 ? 4u : 2u);
    if (per_token > UINT32_MAX || page_bytes % per_token != 0) return 1;
    uint32_t tokens_per_page = page_bytes / (uint32_t)per_token;
    uint32_t group = num_q_heads / num_kv_heads;
    int profile_ok = (head_dim == 128 && tokens_per_page == 8) ||
                     (head_dim == 256 && (tokens_per_page == 8 || tokens_per_page == 16));
    int supports_tiled = !dspark_history && io_dtype == PSI_O_BF16 && profile_ok && group <= 8;
    int full_group = !dspark_history && head_dim == 128 && tokens_per_page == 8;
    uint32_t bounded = head_dim < 256 ? head_dim : 256;
    uint32_t threads = next_pow2_u32(bounded < 32 ? 32 : bounded);
    uint32_t tiled_q_tile = 8;
    uint32_t max_head_tile = 256 / (tiled_q_tile / 8 * 32);
    if (max_q_tokens_per_partial) *max_q_tokens_per_partial = supports_tiled ? tiled_q_tile : 1;
    if (num_tokens == 0 || num_q_token_tiles == 0 || num_q_token_tiles > num_tokens) return 1;
    if (!supports_tiled || (uint64_t)num_tokens < 2ull * num_q_token_tiles) {
        out->tiled_q = 0;
        out->q_token_tile_size = 0;
        out->kv_token_tile_size = threads;
        out->num_threads_per_threadblock = threads;
        out->q_head_tile_size = group < max_head_tile ? group : max_head_tile;
        return 0;
    }
    uint32_t desired = (!full_group && (uint64_t)num_tokens < 4ull * num_q_token_tiles) ? (group + 1) / 2 : group;
    out->tiled_q = 1;
    out->q_token_tile_size = tiled_q_tile;
    out->kv_token_tile_size = 16;
    out->num_threads_per_threadblock = 0;
    out->q_head_tile_size = desired < max_head_tile ? desired : max_head_tile;
    return 0;
}

/* ------------------------------------------------------------------ */
/* Batch metadata / KV-split planner                                   */
/* ------------------------------------------------------------------ */

static uint64_t div_ceil_u64(uint64_t a, uint64_t b) { return (a + b - 1) / b; }

/* crates/inference-executor-metal/src/attn/gqa/batch_metadata.rs:352-424.
 * kv_splits receives 3 u32 per split, cu_kv_splits num_tokens+1 values.  Returns the split count or -1. */
PSI_ORACLE_API int64_t psi_oracle_build_single_q_kv_splits(const uint32_t* flat_token_indices, uint32_t num_tokens,
                                                           uint32_t kv_token_tile_size, uint64_t max_kv_splits,
                                                           uint32_t* kv_splits, uint32_t* cu_kv_splits) {
    if (num_tokens == 0 || max_kv_splits < num_tokens || kv_token_tile_size == 0) return -1;
    uint64_t* tiles = (uint64_t*)malloc(sizeof(uint64_t) * num_tokens);
    uint64_t* splits = (uint64_t*)malloc(sizeof(uint64_t) * num_tokens);
    for (uint32_t i = 0; i < num_tokens; ++i) {
        tiles[i] = div_ceil_u64((uint64_t)flat_token_indices[i] + 1, kv_token_tile_size);
        splits[i] = 1;
    }
    uint64_t total = num_tokens;
    while (total < max_kv_splits) {
        int64_t best = -1;
        uint64_t best_count = 0;
        for (uint32_t i = 0; i < num_tokens; ++i) {
            if (splits[i] < tiles[i]) {
                uint64_t per_split = div_ceil_u64(tiles[i], splits[i]);
                if (best < 0 || per_split > best_count) {
                    best = i;
                    best_count = per_split;
                }
            }
        }
        if (best < 0) break;
        splits[best] += 1;
        total += 1;
    }
    uint64_t n = 0;
    cu_kv_splits[0] = 0;
    for (uint32_t i = 0; i < num_tokens; ++i) {
        uint32_t context_len = flat_token_indices[i] + 1;
        for (uint64_t s = 0; s < splits[i]; ++s) {
            uint64_t tile_begin = tiles[i] * s / splits[i];
            uint64_t tile_end = tiles[i] * (s + 1) / splits[i];
            uint64_t kv_begin = tile_begin * kv_token_tile_size;
            uint64_t kv_end = tile_end * kv_token_tile_size;
            kv_splits[n * 3 + 0] = i;
            kv_splits[n * 3 + 1] = (uint32_t)kv_begin;
            kv_splits[n * 3 + 2] = kv_end < context_len ? (uint32_t)kv_end : context_len;
            ++n;
        }
        cu_kv_splits[i + 1] = (uint32_t)n;
    }
    free(tiles);
    free(splits);
    return (int64_t)n;
}

/* batch_metadata.rs:433-523.  q_token_tiles receives 2 u32 per tile.  *num_tiles_out <- tile count.  Returns the
 * split count or -1. */
PSI_ORACLE_API int64_t psi_oracle_build_tiled_q_kv_splits(const uint32_t* token_indices, const uint32_t* cu_tokens,
                                                          uint32_t num_reqs, uint32_t q_token_tile_size,
                                                          uint32_t kv_token_tile_size, uint64_t max_partial_tokens,
                                                          uint32_t* q_token_tiles, uint32_t* kv_splits,
                                                          uint32_t* cu_kv_splits, uint32_t* num_tiles_out) {
    if (q_token_tile_size == 0 || kv_token_tile_size == 0) return -1;
    uint64_t cap = 0;
    for (uint32_t r = 0; r < num_reqs; ++r) cap += div_ceil_u64(cu_tokens[r + 1] - cu_tokens[r], q_token_tile_size);
    if (cap == 0) return -1;
    uint32_t* t_start = (uint32_t*)malloc(sizeof(uint32_t) * cap);
    uint32_t* t_end = (uint32_t*)malloc(sizeof(uint32_t) * cap);
    uint32_t* t_ctx = (uint32_t*)malloc(sizeof(uint32_t) * cap);
    uint64_t* t_splits = (uint64_t*)malloc(sizeof(uint64_t) * cap);
    uint64_t nt = 0;
    for (uint32_t r = 0; r < num_reqs; ++r) {
        uint32_t req_start = cu_tokens[r], req_end = cu_tokens[r + 1];
        uint32_t start = req_start;
        while (start < req_end) {
            uint32_t len = req_end - start < q_token_tile_size ? req_end - start : q_token_tile_size;
            t_start[nt] = start;
            t_end[nt] = start + len;
            t_ctx[nt] = token_indices[r] + (start + len - req_start);
            t_splits[nt] = 1;
            ++nt;
            start += len;
        }
    }
    uint64_t partial_tokens = 0;
    for (uint64_t i = 0; i < nt; ++i) partial_tokens += t_end[i] - t_start[i];
    int64_t result = -1;
    if (partial_tokens <= max_partial_tokens) {
        while (partial_tokens < max_partial_tokens) {
            int64_t best = -1;
            uint64_t best_count = 0;
            for (uint64_t i = 0; i < nt; ++i) {
                uint64_t len = t_end[i] - t_start[i];
                if (partial_tokens + len > max_partial_tokens) continue;
                uint64_t tiles = div_ceil_u64(t_ctx[i], kv_token_tile_size);
                if (t_splits[i] >= tiles) continue;
                uint64_t per_split = div_ceil_u64(tiles, t_splits[i]);
                if (best < 0 || per_split > best_count) {
                    best = (int64_t)i;
                    best_count = per_split;
                }
            }
            if (best < 0) break;
            partial_tokens += t_end[best] - t_start[best];
            t_splits[best] += 1;
        }
        uint64_t n = 0;
        cu_kv_splits[0] = 0;
        for (uint64_t i = 0; i < nt; ++i) {
            q_token_tiles[i * 2] = t_start[i];
            q_token_tiles[i * 2 + 1] = t_end[i];
            uint64_t tiles = div_ceil_u64(t_ctx[i], kv_token_tile_size);
            for (uint64_t s = 0; s < t_splits[i]; ++s) {
                uint64_t kv_begin = tiles * s / t_splits[i] * kv_token_tile_size;
                uint64_t kv_end = tiles * (s + 1) / t_splits[i] * kv_token_tile_size;
                kv_splits[n * 3] = (uint32_t)i;
                kv_splits[n * 3 + 1] = (uint32_t)kv_begin;
                kv_splits[n * 3 + 2] = kv_end < t_ctx[i] ? (uint32_t)kv_end : t_ctx[i];
                ++n;
            }
            cu_kv_splits[i + 1] = (uint32_t)n;
        }
        *num_tiles_out = (uint32_t)nt;
        result = (int64_t)n;
    }
    free(t_start);
    free(t_end);
    free(t_ctx);
    free(t_splits);
    return result;
}

typedef struct {
    uint32_t num_tokens;
    uint32_t num_total_tokens;
    uint32_t num_q_token_tiles;
    uint32_t num_total_q_token_tiles;
    uint32_t num_sdpa_map_task_templates;
    uint32_t num_total_sdpa_map_task_templates;
    uint32_t reduce_sdpa_partial_outputs;
} psi_oracle_replay_shape;

enum { PSI_O_CAP_EXACT = 0, PSI_O_CAP_BUCKETED = 1, PSI_O_CAP_CALLER_TOKENS = 2 };

/* GQAMetadataBuffers::update_with_capacity (batch_metadata.rs:192-317).  The five arrays are the caller's
 * capacity-sized buffers (max_tokens, max_tokens, 2*max_tokens, 3*max_tokens, max_tokens+1 u32) and are updated in
 * place exactly as the reference writes them: only the active prefix (plus the u32::MAX split padding up to the
 * replay capacity) changes.  Returns 0, or a positive code naming the violated assertion. */
PSI_ORACLE_API int psi_oracle_metadata_update(uint32_t max_tokens, const uint32_t* req_slots,
                                              const uint32_t* token_indices, const uint32_t* cu_tokens,
                                              uint32_t num_reqs, const psi_oracle_variant* variant, int capacity_mode,
                                              const uint32_t* token_topology_boundaries, uint32_t num_boundaries,
                                              uint32_t caller_num_total_tokens, uint32_t* buf_req_slots,
                                              uint32_t* buf_flat_token_indices, uint32_t* buf_q_token_tiles,
                                              uint32_t* buf_kv_splits, uint32_t* buf_cu_kv_splits,
                                              psi_oracle_replay_shape* shape) {
    if (num_reqs == 0 || cu_tokens[0] != 0) return 1;
    for (uint32_t r = 0; r < num_reqs; ++r) {
        if (cu_tokens[r] > cu_tokens[r + 1]) return 2;
        if ((uint64_t)token_indices[r] + (cu_tokens[r + 1] - cu_tokens[r]) > UINT32_MAX) return 3;
    }
    uint32_t num_tokens = cu_tokens[num_reqs];
    if (num_tokens == 0) return 4;
    if (num_tokens > max_tokens) return 5;
    if (capacity_mode == PSI_O_CAP_CALLER_TOKENS) {
        if (num_tokens > caller_num_total_tokens) return 6; /* active token count exceeds caller-owned capacity */
        if (caller_num_total_tokens > max_tokens) return 7; /* caller-owned capacity exceeds metadata capacity */
    }
    uint32_t t = 0;
    for (uint32_t r = 0; r < num_reqs; ++r) {
        for (uint32_t i = 0; i < cu_tokens[r + 1] - cu_tokens[r]; ++i) {
            buf_req_slots[t] = req_slots[r];
            buf_flat_token_indices[t] = token_indices[r] + i;
            ++t;
        }
    }
    uint64_t max_kv_splits = max_tokens;
    uint32_t* splits = (uint32_t*)malloc(sizeof(uint32_t) * 3 * (size_t)max_tokens);
    uint32_t* cu = (uint32_t*)malloc(sizeof(uint32_t) * ((size_t)max_tokens + 1));
    uint32_t* tiles = (uint32_t*)malloc(sizeof(uint32_t) * 2 * (size_t)max_tokens);
    int64_t num_splits;
    uint32_t num_tiles;
    if (!variant->tiled_q) {
        num_splits = psi_oracle_build_single_q_kv_splits(buf_flat_token_indices, num_tokens,
                                                         variant->kv_token_tile_size, max_kv_splits, splits, cu);
        num_tiles = num_tokens;
    } else {
        num_splits = psi_oracle_build_tiled_q_kv_splits(token_indices, cu_tokens, num_reqs, variant->q_token_tile_size,
                                                        variant->kv_token_tile_size, max_tokens, tiles, splits, cu,
                                                        &num_tiles);
    }
    int rc = 0;
    if (num_splits < 0) {
        rc = 8;
    } else {
        uint32_t total_tokens, total_tiles, total_splits;
        uint32_t* buckets = NULL;
        if (capacity_mode == PSI_O_CAP_EXACT) {
            uint64_t p2 = next_pow2_u32((uint32_t)num_splits);
            total_splits = (uint32_t)(p2 < max_kv_splits ? p2 : max_kv_splits);
            total_tokens = num_tokens;
            total_tiles = num_tiles;
        } else {
            /* GQAReplayBucketPolicy (batch_metadata.rs:13-58): token buckets honour the topology boundaries, the
             * tile and split buckets do not. */
            size_t cap = 4096 + (size_t)num_boundaries;
            buckets = (uint32_t*)malloc(sizeof(uint32_t) * cap);
            int64_t nb = psi_oracle_bucket_policy(max_tokens, NULL, 0, buckets, cap);
            total_tiles = psi_oracle_bucket_capacity(buckets, (uint64_t)nb, num_tiles);
            total_splits = psi_oracle_bucket_capacity(buckets, (uint64_t)nb, (uint32_t)num_splits);
            if (capacity_mode == PSI_O_CAP_BUCKETED) {
                nb = psi_oracle_bucket_policy(max_tokens, token_topology_boundaries, num_boundaries, buckets, cap);
                total_tokens = psi_oracle_bucket_capacity(buckets, (uint64_t)nb, num_tokens);
            } else {
                total_tokens = caller_num_total_tokens;
            }
            free(buckets);
        }
        if (total_splits < (uint32_t)num_splits) {
            rc = 9;
        } else {
            if (variant->tiled_q) memcpy(buf_q_token_tiles, tiles, sizeof(uint32_t) * 2 * num_tiles);
            memcpy(buf_kv_splits, splits, sizeof(uint32_t) * 3 * (size_t)num_splits);
            for (size_t i = (size_t)num_splits * 3; i < (size_t)total_splits * 3; ++i) buf_kv_splits[i] = UINT32_MAX;
            memcpy(buf_cu_kv_splits, cu, sizeof(uint32_t) * ((size_t)num_tiles + 1));
            shape->num_tokens = num_tokens;
            shape->num_total_tokens = total_tokens;
            shape->num_q_token_tiles = num_tiles;
            shape->num_total_q_token_tiles = total_tiles;
            shape->num_sdpa_map_task_templates = (uint32_t)num_splits;
            shape->num_total_sdpa_map_task_templates = total_splits;
            shape->reduce_sdpa_partial_outputs = (variant->tiled_q || (uint32_t)num_splits > num_tokens) ? 1u : 0u;
        }
    }
    free(splits);
    free(cu);
    free(tiles);
    return rc;
}

/* ------------------------------------------------------------------ */
/* Page-ID allocator                                                   */
/* ------------------------------------------------------------------ */

/* Single-threaded restatement of U32IDAllocator's observable behaviour: freed IDs are re-issued first, in FIFO order
 * (crossbeam SegQueue), then fresh IDs from a bump counter; a bitmap tracks live IDs.
 * crates/inference-runtime-core/src/memory/u32_id_allocator.rs:69-172 */
typedef struct {
    uint64_t capacity;
    uint32_t counter;
    uint32_t* queue; /* ring buffer of freed ids, capacity+1 slots */
    uint64_t q_head, q_len;
    uint64_t* bitmap;
    uint64_t num_words;
} psi_oracle_allocator;

PSI_ORACLE_API psi_oracle_allocator* psi_oracle_allocator_new(uint64_t capacity) {
    if (capacity > UINT32_MAX) return NULL;
    psi_oracle_allocator* a = (psi_oracle_allocator*)calloc(1, sizeof(*a));
    a->capacity = capacity;
    a->queue = (uint32_t*)malloc(sizeof(uint32_t) * (capacity + 1));
    a->num_words = (capacity + 63) / 64;
    a->bitmap = (uint64_t*)calloc(a->num_words ? a->num_words : 1, sizeof(uint64_t));
    return a;
}

PSI_ORACLE_API void psi_oracle_allocator_free(psi_oracle_allocator* a) {
    if (!a) return;
    free(a->queue);
    free(a->bitmap);
    free(a);
}

static void alloc_mark(psi_oracle_allocator* a, uint32_t id, int live) {
    if (live) a->bitmap[id >> 6] |= 1ull << (id & 63); else a->bitmap[id >> 6] &= ~(1ull << (id & 63));
}

static int queue_pop(psi_oracle_allocator* a, uint32_t* id) {
    if (a->q_len == 0) return 0;
    *id = a->queue[a->q_head];
    a->q_head = (a->q_head + 1) % (a->capacity + 1);
    a->q_len -= 1;
    return 1;
}

static void queue_push(psi_oracle_allocator* a, uint32_t id) {
    a->queue[(a->q_head + a->q_len) % (a->capacity + 1)] = id;
    a->q_len += 1;
}

/* u32_id_allocator.rs:107-144.  Returns 0 and fills ids, or 1 ("not enough ID") leaving the allocator unchanged
 * except that popped free IDs return to the back of the queue, as in the reference. */
PSI_ORACLE_API int psi_oracle_allocator_alloc_many(psi_oracle_allocator* a, uint64_t count, uint32_t* ids) {
    uint64_t n = 0;
    while (n < count && queue_pop(a, &ids[n])) ++n;
    if (n < count) {
        uint64_t fresh = count - n;
        uint64_t end = (uint64_t)a->counter + fresh;
        if (end > a->capacity) {
            for (uint64_t i = 0; i < n; ++i) queue_push(a, ids[i]);
            return 1;
        }
        for (uint64_t i = 0; i < fresh; ++i) ids[n + i] = a->counter + (uint32_t)i;
        a->counter = (uint32_t)end;
    }
    for (uint64_t i = 0; i < count; ++i) alloc_mark(a, ids[i], 1);
    return 0;
}

PSI_ORACLE_API int psi_oracle_allocator_alloc_one(psi_oracle_allocator* a, uint32_t* id) {
    return psi_oracle_allocator_alloc_many(a, 1, id);
}

PSI_ORACLE_API void psi_oracle_allocator_free_many(psi_oracle_allocator* a, const uint32_t* ids, uint64_t count) {
    for (uint64_t i = 0; i < count; ++i) {
        alloc_mark(a, ids[i], 0);
        queue_push(a, ids[i]);
    }
}

PSI_ORACLE_API uint64_t psi_oracle_allocator_bitmap(const psi_oracle_allocator* a, uint64_t* words, uint64_t cap) {
    for (uint64_t i = 0; i < a->num_words && i < cap; ++i) words[i] = a->bitmap[i];
    return a->num_words;
}

PSI_ORACLE_API uint64_t psi_oracle_allocator_free_count(const psi_oracle_allocator* a) {
    return a->q_len + (a->capacity - a->counter);
}

/* ------------------------------------------------------------------ */
/* Neighbours of the path: q/k RMSNorm + RoPE, attention-output gate   */
/* ------------------------------------------------------------------ */

typedef struct {
    uint32_t enabled;  /* 0 = RopeScaling::Default */
    float factor;
    float attention_factor;
    float beta_fast;
    float beta_slow;
    uint32_t original_max_position_embeddings;
    uint32_t truncate;
} psi_oracle_yarn;

/* RopeScaling::kernel_parameters / yarn_kernel_parameters,
 * crates/inference-backend-metal/src/components/rms_norm_rope.rs:167-230.  Writes rope_dim/2 inverse frequencies,
 * the attention factor and (when yarn is on) the correction range. */
PSI_ORACLE_API int psi_oracle_rope_parameters(uint32_t rope_dim, float rope_theta, const psi_oracle_yarn* yarn,
                                              float* inverse_frequencies, float* attention_factor,
                                              float* correction_low, float* correction_high) {
    uint32_t rope_half = rope_dim / 2;
    float low = 0.0f, high = 0.0f;
    int on = yarn != NULL && yarn->enabled;
    if (on) {
        double dimension = (double)rope_dim, base = (double)rope_theta;
        double original = (double)yarn->original_max_position_embeddings;
        float c_fast = (float)(dimension * log(original / ((double)yarn->beta_fast * 6.283185307179586)) / (2.0 * log(base)));
        float c_slow = (float)(dimension * log(original / ((double)yarn->beta_slow * 6.283185307179586)) / (2.0 * log(base)));
        low = c_fast > 0.0f ? c_fast : 0.0f;
        float cap = rope_dim > 0 ? (float)(rope_dim - 1) : 0.0f;
        high = c_slow < cap ? c_slow : cap;
        if (yarn->truncate) {
            low = floorf(low);
            high = ceilf(high);
        }
        if (!(low <= high)) return 1;
        if (low == high) high += 0.001f;
    }
    for (uint32_t d = 0; d < rope_half; ++d) {
        float inv = powf(rope_theta, -((float)d / (float)rope_half));
        if (on) {
            float ramp = ((float)d - low) / (high - low);
            ramp = ramp < 0.0f ? 0.0f : (ramp > 1.0f ? 1.0f : ramp);
            inv *= 1.0f + ramp * (1.0f / yarn->factor - 1.0f);
        }
        if (!(inv > 0.0f) || !isfinite(inv)) return 2;
        inverse_frequencies[d] = inv;
    }
    *attention_factor = on ? yarn->attention_factor : 1.0f;
    if (correction_low) *correction_low = low;
    if (correction_high) *correction_high = high;
    return 0;
}

/* Round-trip through the storage dtype T (identity for f32): the shader's T(...) casts. */
static inline float round_to(float v, int dtype) {
    if (dtype == PSI_O_F32) return v;
    if (dtype == PSI_O_BF16) return psi_oracle_bf16_to_f32(psi_oracle_f32_to_bf16(v));
    return psi_oracle_f16_to_f32(psi_oracle_f32_to_f16(v));
}

static inline void store_elem(void* base, size_t index, int dtype, float v) {
    if (dtype == PSI_O_F32) ((float*)base)[index] = v;
    else if (dtype == PSI_O_BF16) ((uint16_t*)base)[index] = psi_oracle_f32_to_bf16(v);
    else ((uint16_t*)base)[index] = psi_oracle_f32_to_f16(v);
}

/* Per (token, head) row: RMS-normalise, scale by the bf16 weight with the shader's rounding order
 * (T(weight) * T(x * inv_rms)), rotate the first rope_dim dims by position * inverse_frequency.
 * crates/inference-backend-metal/src/components/metal/rms_norm_rope.metal:7-82; the row sum is taken sequentially in
 * f32 as the reference's own CPU expectations do (rms_norm_rope.rs:448-450,500-507). */
PSI_ORACLE_API void psi_oracle_rms_norm_rope(const void* input, int dtype, const uint16_t* norm_weight_bf16,
                                             const uint32_t* flat_token_indices, uint32_t num_tokens,
                                             uint32_t num_heads, uint32_t head_dim, uint32_t rope_dim, float eps,
                                             const float* inverse_frequencies, float attention_factor, void* output) {
    uint32_t rope_half = rope_dim / 2;
    for (uint32_t row = 0; row < num_tokens * num_heads; ++row) {
        size_t base = (size_t)row * head_dim;
        float acc = 0.0f;
        for (uint32_t d = 0; d < head_dim; ++d) {
            float x = load_elem(input, base + d, dtype);
            acc += x * x;
        }
        float inv_rms = 1.0f / sqrtf(acc / (float)head_dim + eps);
        float position = (float)flat_token_indices[row / num_heads];
        for (uint32_t d = 0; d < head_dim; ++d) {
            float w = round_to(psi_oracle_bf16_to_f32(norm_weight_bf16[d]), dtype);
            float xn = round_to(w * round_to(load_elem(input, base + d, dtype) * inv_rms, dtype), dtype);
            if (d < rope_half) {
                uint32_t d2 = d + rope_half;
                float w2 = round_to(psi_oracle_bf16_to_f32(norm_weight_bf16[d2]), dtype);
                float x2 = round_to(w2 * round_to(load_elem(input, base + d2, dtype) * inv_rms, dtype), dtype);
                float theta = position * inverse_frequencies[d];
                float c = cosf(theta), s = sinf(theta);
                store_elem(output, base + d, dtype, attention_factor * (xn * c - x2 * s));
                store_elem(output, base + d2, dtype, attention_factor * (xn * s + x2 * c));
            } else if (d >= rope_dim) {
                store_elem(output, base + d, dtype, xn);
            }
        }
    }
}

/* De-interleave of the fused projection output, one element at a time as the shaders do.  gated != 0:
 * per token Hq pairs (q[D] | g[D]), then Hkv k rows, then Hkv v rows
 * (crates/inference-backend-metal/src/components/metal/gqa_qgkv_split.metal:14-42); gated == 0: q rows, k rows, v rows
 * and no g (metal/gqa_qkv_split.metal:13-36).  Elements are moved as bits (elem_bytes = 2 or 4). */
PSI_ORACLE_API void psi_oracle_projection_split(const void* projection, uint32_t elem_bytes, uint32_t gated,
                                                uint32_t num_tokens, uint32_t num_q_heads, uint32_t num_kv_heads,
                                                uint32_t head_dim, void* q, void* g, void* k, void* v) {
    const size_t q_slots = (size_t)num_q_heads * head_dim, kv_slots = (size_t)num_kv_heads * head_dim;
    const size_t token_width = (gated ? 2 : 1) * q_slots + 2 * kv_slots;
    const unsigned char* src = (const unsigned char*)projection;
    for (size_t gid = 0; gid < (size_t)num_tokens * token_width; ++gid) {
        const size_t token = gid / token_width;
        size_t slot = gid - token * token_width;
        unsigned char* dst;
        size_t index;
        if (gated && slot < 2 * q_slots) {
            const size_t pair = slot / (2 * (size_t)head_dim), in_pair = slot - pair * 2 * head_dim;
            index = (token * num_q_heads + pair) * head_dim + in_pair % head_dim;
            dst = (unsigned char*)(in_pair < head_dim ? q : g);
        } else if (!gated && slot < q_slots) {
            index = token * q_slots + slot;
            dst = (unsigned char*)q;
        } else {
            slot -= (gated ? 2 : 1) * q_slots;
            if (slot < kv_slots) {
                index = token * kv_slots + slot;
                dst = (unsigned char*)k;
            } else {
                index = token * kv_slots + (slot - kv_slots);
                dst = (unsigned char*)v;
            }
        }
        memcpy(dst + index * elem_bytes, src + gid * elem_bytes, elem_bytes);
    }
}

/* out = attention_output * sigmoid(gate) with the shader's per-dtype arithmetic: f32 throughout, or every step
 * rounded to bf16.  crates/inference-backend-metal/src/components/metal/gqa_activation_gate.metal:5-39 */
PSI_ORACLE_API void psi_oracle_activation_gate(const void* attention_output, const void* gates, int dtype, size_t n,
                                               void* output) {
    for (size_t i = 0; i < n; ++i) {
        float a = load_elem(attention_output, i, dtype), x = load_elem(gates, i, dtype);
        float sig;
        if (dtype == PSI_O_F32) {
            float y = 1.0f / (1.0f + expf(-fabsf(x)));
            sig = x < 0.0f ? 1.0f - y : y;
        } else {
            float abs_x = round_to(fabsf(x), dtype);
            float exp_x = round_to(expf(round_to(-abs_x, dtype)), dtype);
            float denom = round_to(1.0f + exp_x, dtype);
            float y = round_to(1.0f / denom, dtype);
            sig = x < 0.0f ? round_to(1.0f - y, dtype) : y;
        }
        store_elem(output, i, dtype, a * sig);
    }
}

/* Dense bidirectional attention of every query token against the tokens of its own block of `block_size` tokens
 * (local, unpaged K/V), as a partial in the reduce's ABI: normalised output, natural-log max, exp-sum per
 * (token, q head).  crates/inference-backend-metal/src/components/metal/gqa_block_sdpa.metal:5-77 and the reference
 * computation of crates/inference-backend-metal/src/components/gqa_block_attention_test.rs:98-139.
 * q [T][Hq][D], local_k / local_v [T][Hkv][D] in `dtype`; partial_output [T][Hq][D] f32 (unrounded), partial_max and
 * partial_sum [T][Hq]. */
PSI_ORACLE_API void psi_oracle_block_sdpa(const void* q, const void* local_k, const void* local_v, int dtype,
                                          uint32_t num_tokens, uint32_t block_size, uint32_t num_q_heads,
                                          uint32_t num_kv_heads, uint32_t head_dim, float scale, float* partial_output,
                                          float* partial_max, float* partial_sum) {
    uint32_t group = num_q_heads / num_kv_heads;
    float* weights = (float*)malloc(sizeof(float) * block_size);
    for (uint32_t t = 0; t < num_tokens; ++t) {
        uint32_t begin = t / block_size * block_size;
        for (uint32_t h = 0; h < num_q_heads; ++h) {
            uint32_t kv_head = h / group;
            size_t q_row = ((size_t)t * num_q_heads + h) * head_dim;
            float max_logit = -INFINITY;
            for (uint32_t j = 0; j < block_size; ++j) {
                size_t k_row = ((size_t)(begin + j) * num_kv_heads + kv_head) * head_dim;
                float score = 0.0f;
                for (uint32_t d = 0; d < head_dim; ++d) score += load_elem(q, q_row + d, dtype) * load_elem(local_k, k_row + d, dtype);
                weights[j] = score * scale;
                if (weights[j] > max_logit) max_logit = weights[j];
            }
            float exp_sum = 0.0f;
            for (uint32_t j = 0; j < block_size; ++j) {
                weights[j] = expf(weights[j] - max_logit);
                exp_sum += weights[j];
            }
            size_t out_row = (size_t)t * num_q_heads + h;
            partial_max[out_row] = max_logit;
            partial_sum[out_row] = exp_sum;
            for (uint32_t d = 0; d < head_dim; ++d) {
                float acc = 0.0f;
                for (uint32_t j = 0; j < block_size; ++j) {
                    size_t v_row = ((size_t)(begin + j) * num_kv_heads + kv_head) * head_dim;
                    acc += weights[j] * load_elem(local_v, v_row + d, dtype);
                }
                partial_output[out_row * head_dim + d] = exp_sum > 0.0f ? acc / exp_sum : 0.0f;
            }
        }
    }
    free(weights);
}
