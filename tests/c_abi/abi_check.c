/*
 * A C11 caller of include/psi_cuda.h and nothing else: what a binding in another language (the Rust crate
 * inference-backend-cuda, cgo, JNI) sees of the library.
 *
 *   abi_check layout            prints sizeof and offsetof of every struct that crosses the boundary, one per line,
 *                               so that the ctypes mirror and the #[repr(C)] blocks of INTEGRATION.md can be held
 *                               against what the compiler laid out (no GPU needed)
 *   abi_check step <out.bin>    runs the CPU-scale configuration end to end on device 0 (batch 1, 4 Q heads / 1 KV head,
 *                               head_dim 128, fp16, 256 cached tokens in 16-token pages of a 64-page arena, one token
 *                               appended at position 256, attention over 257 keys) through the calls the reference's
 *                               GQA::record order stands for, and writes q | k | v | arena after the step | out as raw
 *                               bytes for the caller to check
 *
 * Inputs come from a 32-bit LCG so that any language can regenerate them: state = state * 1664525 + 1013904223,
 * value = ((state >> 8) / 2^24) * 2 - 1, the generator of the reference's parity fixtures
 * (crates/inference-backend-metal/src/components/gqa_split_kv_single_q_test.rs:432-440), rounded to fp16 by truncation
 * of a float's bits here (exact conversion is not the point of this program; the checker reads the fp16 bits back).
 */
#include <stddef.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "psi_cuda.h"

#define FIELD(type, field) printf(#type "." #field " offset %zu size %zu\n", offsetof(type, field), sizeof(((type*)0)->field))
#define WHOLE(type) printf(#type " sizeof %zu\n", sizeof(type))

static void print_layout(void) {
    WHOLE(psi_page_table_layout);
    FIELD(psi_page_table_layout, num_req_slots);
    FIELD(psi_page_table_layout, num_gqa_layers);
    FIELD(psi_page_table_layout, num_blocks);
    FIELD(psi_page_table_layout, num_page_ids_per_block);
    WHOLE(psi_replay_shape);
    FIELD(psi_replay_shape, num_tokens);
    FIELD(psi_replay_shape, num_total_tokens);
    FIELD(psi_replay_shape, num_q_token_tiles);
    FIELD(psi_replay_shape, num_total_q_token_tiles);
    FIELD(psi_replay_shape, num_sdpa_map_task_templates);
    FIELD(psi_replay_shape, num_total_sdpa_map_task_templates);
    FIELD(psi_replay_shape, reduce_sdpa_partial_outputs);
    WHOLE(psi_split_kv_variant);
    FIELD(psi_split_kv_variant, tiled_q);
    FIELD(psi_split_kv_variant, q_token_tile_size);
    FIELD(psi_split_kv_variant, kv_token_tile_size);
    FIELD(psi_split_kv_variant, num_threads_per_threadblock);
    FIELD(psi_split_kv_variant, q_head_tile_size);
    WHOLE(psi_norm_rope_config);
    FIELD(psi_norm_rope_config, rope_dim);
    FIELD(psi_norm_rope_config, eps);
    FIELD(psi_norm_rope_config, rope_theta);
    FIELD(psi_norm_rope_config, yarn_enabled);
    FIELD(psi_norm_rope_config, yarn_factor);
    FIELD(psi_norm_rope_config, yarn_attention_factor);
    FIELD(psi_norm_rope_config, yarn_beta_fast);
    FIELD(psi_norm_rope_config, yarn_beta_slow);
    FIELD(psi_norm_rope_config, yarn_original_max_position_embeddings);
    FIELD(psi_norm_rope_config, yarn_truncate);
    WHOLE(psi_gqa_config);
    FIELD(psi_gqa_config, num_q_heads);
    FIELD(psi_gqa_config, num_kv_heads);
    FIELD(psi_gqa_config, head_dim);
    FIELD(psi_gqa_config, scale);
    FIELD(psi_gqa_config, page_bytes);
    FIELD(psi_gqa_config, dtype);
    FIELD(psi_gqa_config, layout);
    FIELD(psi_gqa_config, max_tokens);
    FIELD(psi_gqa_config, plan_mode);
    FIELD(psi_gqa_config, kernel_mode);
    FIELD(psi_gqa_config, max_ctas);
    WHOLE(psi_u32_range);
    FIELD(psi_u32_range, begin);
    FIELD(psi_u32_range, end);
    WHOLE(psi_hibernation_plan);
    FIELD(psi_hibernation_plan, selected);
    FIELD(psi_hibernation_plan, request_slot_ranges);
    FIELD(psi_hibernation_plan, num_request_slot_ranges);
    FIELD(psi_hibernation_plan, page_id_ranges);
    FIELD(psi_hibernation_plan, num_page_id_ranges);
    WHOLE(psi_kv_exchange);
    FIELD(psi_kv_exchange, rank);
    FIELD(psi_kv_exchange, world);
    FIELD(psi_kv_exchange, owner);
    FIELD(psi_kv_exchange, step);
    FIELD(psi_kv_exchange, slots);
    FIELD(psi_kv_exchange, slot_floats);
    FIELD(psi_kv_exchange, flags);
    FIELD(psi_kv_exchange, consumed);
    FIELD(psi_kv_exchange, max_polls);
    printf("enum PSI_ERR_PAGE_ID %d PSI_DTYPE_F16 %d PSI_KERNEL_MMA_SYNC %d PSI_CAPACITY_CALLER_TOKENS %d PSI_MD_CU_KV_SPLITS %d "
           "PSI_SNAPSHOT_DSPARK_GQA_REQUEST_PAGE_TABLE %d\n",
           (int)PSI_ERR_PAGE_ID, (int)PSI_DTYPE_F16, (int)PSI_KERNEL_MMA_SYNC, (int)PSI_CAPACITY_CALLER_TOKENS,
           (int)PSI_MD_CU_KV_SPLITS, (int)PSI_SNAPSHOT_DSPARK_GQA_REQUEST_PAGE_TABLE);
    printf("define PSI_STATIC_MAX_HEAD_DIM %d PSI_STATIC_MAX_CTAS %d PSI_STATIC_MAX_ITEMS %d PSI_STATIC_SCRATCH_BYTES %d\n",
           PSI_STATIC_MAX_HEAD_DIM, PSI_STATIC_MAX_CTAS, PSI_STATIC_MAX_ITEMS, PSI_STATIC_SCRATCH_BYTES);
}

static uint32_t lcg_state = 0x4C8F17D2u;

static float lcg_next(void) {
    lcg_state = lcg_state * 1664525u + 1013904223u;
    return (float)(lcg_state >> 8) / 16777216.0f * 2.0f - 1.0f;
}

/* float -> IEEE half, round toward zero; enough for values in (-1, 1) */
static uint16_t to_half(float f) {
    uint32_t x;
    memcpy(&x, &f, sizeof x);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const int32_t exponent = (int32_t)((x >> 23) & 0xFFu) - 127 + 15;
    const uint32_t mantissa = x & 0x7FFFFFu;
    if (exponent <= 0) return (uint16_t)sign; /* flush tiny values to zero */
    if (exponent >= 31) return (uint16_t)(sign | 0x7BFFu);
    return (uint16_t)(sign | ((uint32_t)exponent << 10) | (mantissa >> 13));
}

#define CHECK(call)                                                                        \
    do {                                                                                   \
        const int32_t status_ = (call);                                                    \
        if (status_ != PSI_OK) {                                                           \
            char message_[512] = "";                                                       \
            if (ctx != NULL) psi_ctx_last_error(ctx, message_, sizeof message_);           \
            if (message_[0] == '\0') psi_last_error(message_, sizeof message_);            \
            fprintf(stderr, "%s failed with status %d: %s\n", #call, status_, message_);   \
            return 1;                                                                      \
        }                                                                                  \
    } while (0)

static int run_step(const char* out_path) {
    enum { HQ = 4, HKV = 1, D = 128, P = 16, PAGES = 64, CONTEXT = 256 };
    const uint32_t page_bytes = 2u * HKV * P * D * 2u;
    const size_t page_elems = page_bytes / 2u;
    psi_ctx* ctx = NULL;
    psi_pages* pages = NULL;
    psi_table* table = NULL;
    psi_gqa* gqa = NULL;
    CHECK(psi_ctx_create(0, &ctx));
    CHECK(psi_pages_create(ctx, PAGES, page_bytes, &pages));
    const psi_page_table_layout layout = {1, 1, PAGES, 1};
    CHECK(psi_table_create(ctx, &layout, &table));
    CHECK(psi_table_set_page_bound(table, PAGES));

    /* arena contents, then q, k, v, all from the one generator */
    uint16_t* arena = malloc(PAGES * page_elems * sizeof(uint16_t));
    uint16_t q[HQ * D], k[HKV * D], v[HKV * D], out[HQ * D];
    if (arena == NULL) return 1;
    for (size_t i = 0; i < PAGES * page_elems; ++i) arena[i] = to_half(lcg_next());
    for (int i = 0; i < HQ * D; ++i) q[i] = to_half(lcg_next());
    for (int i = 0; i < HKV * D; ++i) k[i] = to_half(lcg_next());
    for (int i = 0; i < HKV * D; ++i) v[i] = to_half(lcg_next());
    CHECK(psi_pages_import_range(pages, 0, PAGES, arena));

    /* block table: logical page i of the request lives in physical page (i * 37 + 11) mod 64, a fixed permutation */
    uint32_t ids[PAGES];
    for (uint32_t i = 0; i < PAGES; ++i) ids[i] = (i * 37u + 11u) % PAGES;
    CHECK(psi_table_write_row(table, 0, 0, ids, PAGES));

    psi_gqa_config config;
    memset(&config, 0, sizeof config);
    config.num_q_heads = HQ;
    config.num_kv_heads = HKV;
    config.head_dim = D;
    config.scale = 0.08838834764831845f; /* 1 / sqrt(128) */
    config.page_bytes = page_bytes;
    config.dtype = PSI_DTYPE_F16;
    config.layout = layout;
    config.max_tokens = 1;
    config.plan_mode = PSI_PLAN_BALANCED;
    config.kernel_mode = PSI_KERNEL_AUTO;
    CHECK(psi_gqa_create(ctx, &config, &gqa));

    const uint32_t req_slots[1] = {0}, token_indices[1] = {CONTEXT}, cu_tokens[2] = {0, 1};
    psi_replay_shape shape;
    CHECK(psi_gqa_prepare(gqa, req_slots, token_indices, cu_tokens, 1, PSI_CAPACITY_EXACT, 0, &shape));
    if (shape.num_tokens != 1) {
        fprintf(stderr, "unexpected replay shape\n");
        return 1;
    }
    /* host buffers in, host buffer out: plan, transfers, append, attention and the result in one blocking call */
    CHECK(psi_gqa_decode_step_host(gqa, pages, table, 0, k, v, q, out));
    int32_t device_status = -1;
    CHECK(psi_gqa_device_status(gqa, &device_status));
    if (device_status != 0) {
        fprintf(stderr, "device status %d\n", device_status);
        return 1;
    }
    CHECK(psi_pages_export_range(pages, 0, PAGES, arena));

    FILE* f = fopen(out_path, "wb");
    if (f == NULL) return 1;
    fwrite(q, sizeof q, 1, f);
    fwrite(k, sizeof k, 1, f);
    fwrite(v, sizeof v, 1, f);
    fwrite(arena, sizeof(uint16_t), PAGES * page_elems, f);
    fwrite(out, sizeof out, 1, f);
    fclose(f);
    free(arena);
    CHECK(psi_gqa_destroy(gqa));
    CHECK(psi_table_destroy(table));
    CHECK(psi_pages_destroy(pages));
    CHECK(psi_ctx_destroy(ctx));
    printf("step ok\n");
    return 0;
}

int main(int argc, char** argv) {
    if (argc >= 2 && strcmp(argv[1], "layout") == 0) {
        print_layout();
        return 0;
    }
    if (argc >= 3 && strcmp(argv[1], "step") == 0) return run_step(argv[2]);
    fprintf(stderr, "usage: abi_check layout | abi_check step <out.bin>\n");
    return 2;
}
