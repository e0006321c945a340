/* TEST INFRASTRUCTURE ONLY.
 *
 * The reference's graph-level attention files (src/graph/core.c, attention.c,
 * numeric.c, plan.c) hold the CPU latent reduce, the sparse index selection,
 * the top-k ranking and the position rotation that the checkers here are
 * pinned against. The same files also hold the model-bound drivers around
 * them, which name functions of the reference's model, runtime-descriptor
 * and materialization layers. Nothing on the call tree of the four entry
 * points the bridge uses (yvex_attention_reduce_chunk, yvex_attention_csa_select,
 * yvex_attention_topk_select, yvex_attention_rope_apply) reaches those
 * functions, so the CPU-only reference build resolves each of them to a
 * stand-in that stops the process if it is ever entered. No reference header
 * is included: the stand-ins are never called through their real signatures.
 */
#include <stdio.h>
#include <stdlib.h>

#define YVX_REF_ABSENT(name)                                                        \
    void name(void)                                                                 \
    {                                                                               \
        fputs("oracle/_ref: " #name " is outside the CPU-only reference build\n",   \
              stderr);                                                              \
        abort();                                                                    \
    }

YVX_REF_ABSENT(yvex_arch_name)
YVX_REF_ABSENT(yvex_attention_comparison_failure_publish)
YVX_REF_ABSENT(yvex_attention_device_completion_resolve)
YVX_REF_ABSENT(yvex_attention_execution_trace_release)
YVX_REF_ABSENT(yvex_attention_publication_identity_build)
YVX_REF_ABSENT(yvex_attention_rolling_storage_acquire)
YVX_REF_ABSENT(yvex_attention_state_provider_abort)
YVX_REF_ABSENT(yvex_attention_state_recipe_seal)
YVX_REF_ABSENT(yvex_attention_workspace_recipe_seal)
YVX_REF_ABSENT(yvex_backend_attention_complete)
YVX_REF_ABSENT(yvex_dtype_tensor_storage_bytes)
YVX_REF_ABSENT(yvex_execution_memory_facts_merge)
YVX_REF_ABSENT(yvex_materialization_session_read)
YVX_REF_ABSENT(yvex_materialization_session_summary)
YVX_REF_ABSENT(yvex_model_activation_identity_update)
YVX_REF_ABSENT(yvex_model_arch)
YVX_REF_ABSENT(yvex_model_context_length)
YVX_REF_ABSENT(yvex_model_name)
YVX_REF_ABSENT(yvex_model_position_identity_update)
YVX_REF_ABSENT(yvex_model_topk_identity_update)
YVX_REF_ABSENT(yvex_runtime_descriptor_find_role)
YVX_REF_ABSENT(yvex_runtime_descriptor_summary_get)
YVX_REF_ABSENT(yvex_runtime_descriptor_tensor_at)
YVX_REF_ABSENT(yvex_semantic_model_ir_attention_view)
YVX_REF_ABSENT(yvex_semantic_model_ir_summary_get)
YVX_REF_ABSENT(yvex_tensor_role_name)
YVX_REF_ABSENT(yvex_tensor_table_at)
YVX_REF_ABSENT(yvex_tensor_table_count)
