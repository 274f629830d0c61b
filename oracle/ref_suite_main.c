/*
 * TEST INFRASTRUCTURE -- not part of the product.
 *
 * Runs test functions of the reference's own suite by name. The reference's
 * tests/test_main.c runs all of them in one process and prints one summary;
 * the acceptance tests of this repository want one test per process (a
 * failed requirement in the reference exits the process) and only the tests
 * that reach the attention path, so this small driver is linked with the
 * reference's unmodified test sources (tests/unit, tests/parity,
 * tests/test_helpers.c) in place of its main.
 *
 *   ref_suite --list              names, one per line
 *   ref_suite NAME [NAME ...]     run them; exit 0 iff all returned 1
 *
 * A name is the reference's function name (tests/test_suite.h) without the
 * leading "run_". FBLT_REF_TEST_DATA overrides the folder the parity tests
 * read their fixtures from (default data/tests, as in the reference).
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "test_suite.h"

const char *g_test_data_dir = "data/tests";

typedef struct {
    const char *name;
    int (*fn)(void);
} suite_entry;

#define T(fn) {#fn, fn}
static const suite_entry k_tests[] = {
    T(run_tensor_core_tests), T(run_json_parser_tests), T(run_allocator_core_tests), T(run_backend_core_tests),
    T(run_cuda_arena_transfer_tests), T(run_elementwise_backend_tests), T(run_gelu_backend_tests),
    T(run_matmul_backend_tests), T(run_matmul_backward_backend_tests), T(run_softmax_backend_tests),
    T(run_cross_entropy_tests), T(run_rope_backend_test), T(run_optim_backend_tests),
    T(run_mask_builder_backend_tests), T(run_entropy_model_tests), T(run_byte_embedding_model_tests),
    T(run_patcher_model_tests), T(run_attention_model_tests), T(run_attention_masked_model_tests),
    T(run_attention_backward_model_tests), T(run_cross_attention_model_tests),
    T(run_cross_attention_masked_model_tests), T(run_cross_attention_backward_model_tests), T(run_elm_model_tests),
    T(run_hash_ngram_model_tests), T(run_lencoder_mask_model_test), T(run_local_encoder_smoke_test),
    T(run_local_encoder_k_split), T(run_global_transformer_causal_mask), T(run_global_transformer_doc_boundary),
    T(run_local_decoder_cross_mask), T(run_local_decoder_paper_rule), T(run_local_decoder_k_split),
    T(run_blt_model_generate_sanity), T(run_model_stage_split_equivalence), T(run_model_multi_doc_isolation),
    T(run_model_decode_nullable_loss), T(run_decoder_d0_modes), T(run_rope_position_gather_test),
    T(run_infer_stats_test), T(run_verify_draft_directed), T(run_selfspec_structural_random),
    T(run_selfspec_equivalence_trained), T(run_kv_cache_logits_equal_dense), T(run_kv_cache_rollback_commit),
    T(run_blockgen_select_kernels), T(run_blockgen_draft_behavior), T(run_blockgen_generation_gates),
    T(run_blockgen_stage6_helpers), T(run_block_diffusion_mask_fixture), T(run_block_diffusion_mask_no_leak),
    T(run_block_diffusion_gradcheck), T(run_block_diffusion_overfit_gate), T(run_block_diffusion_no_label_leak),
    T(run_block_diffusion_last_row_upweight), T(run_block_diffusion_draft_trailing_closed),
    T(run_matmul_parity_test), T(run_softmax_parity_test), T(run_cuda_parity_elementwise),
    T(run_cuda_parity_reductions), T(run_cuda_parity_matmul), T(run_cuda_parity_composites),
    T(run_cuda_parity_training_step), T(run_transformer_parity_tests), T(run_patcher_parity_tests),
    T(run_elm_overfit_tests), T(run_lencoder_overfit_test), T(run_local_encoder_parity),
    T(run_global_transformer_parity), T(run_global_transformer_overfit), T(run_local_decoder_parity),
    T(run_local_decoder_overfit), T(run_blt_model_overfit), T(run_bf16_cast_tests),
    T(run_deterministic_regression_test), T(run_topk_from_logits_tests), T(run_train_window_order_tests),
    T(run_lr_schedule_tests), T(run_decode_select_tests), T(run_patch_capacity_consistency_tests),
};
#undef T
static const size_t k_num_tests = sizeof(k_tests) / sizeof(k_tests[0]);

int main(int argc, char **argv) {
    const char *data = getenv("FBLT_REF_TEST_DATA");
    if (data && *data) g_test_data_dir = data;
    if (argc < 2) {
        fprintf(stderr, "usage: %s --list | NAME [NAME ...]\n", argv[0]);
        return 2;
    }
    if (!strcmp(argv[1], "--list")) {
        for (size_t t = 0; t < k_num_tests; ++t) printf("%s\n", k_tests[t].name + 4);
        return 0;
    }
    int failed = 0;
    for (int a = 1; a < argc; ++a) {
        const suite_entry *e = NULL;
        for (size_t t = 0; t < k_num_tests; ++t)
            if (!strcmp(argv[a], k_tests[t].name + 4)) e = &k_tests[t];
        if (!e) {
            fprintf(stderr, "unknown test '%s'\n", argv[a]);
            return 2;
        }
        const int ok = e->fn();
        printf("[%s] %s\n", ok ? "PASS" : "FAIL", argv[a]);
        fflush(stdout);
        if (!ok) failed++;
    }
    return failed ? 1 : 0;
}
