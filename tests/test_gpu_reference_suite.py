"""The reference's own test suite as the acceptance test of the drop-in operator.

Two executables, built by `make -C oracle accept` from the reference's unmodified sources where
its tree is mounted (outputs under oracle/_ref/, which travel to the GPU box):

* ref_suite_cuda  -- the reference's CUDA backend for sm_100a, minus its attention forward
  operator and its mask-builder file, linked against libfblt_attn.so: core/backend.c:200 binds
  blt_attention_head_core_cuda from the library, core/backend.c:190-192 binds the two mask
  builders from fblt_b200/csrc/blt_backend_glue.c. Its CUDA parity tests compare the CUDA backend
  with the CPU backend inside one process.
* ref_suite_stage -- the reference's CPU build with blt_attention_head_core_cpu replaced by a
  host-staging call into the same library operator (oracle/ref_stage_op.c). The reference's unit
  tests allocate from CPU arenas, so this is how its models, KV cache and generation loops
  (cached == dense logits, BLT-DV == greedy, BLT-S == greedy, the verify-draft cases) run with the
  sm_100a operator underneath. Every call is also checked against the reference's CPU operator.

One test per process: a failed requirement in the reference exits the process.
"""
import os
import re
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
REF = Path(__file__).resolve().parent.parent / "oracle" / "_ref"
STAGE = REF / "ref_suite_stage"
CUDA = REF / "ref_suite_cuda"

# Tests of the reference that reach the attention operator (each name is the reference's function
# in tests/test_suite.h without "run_"), grouped by what they pin.
STAGE_TESTS = [
    # operator through the MHA / cross-attention callers: tests/unit/models/unit_attention.c:10-189,
    # unit_cross_attention.c:20-251 (known-answer constants, mask == is_causal)
    "attention_model_tests", "attention_masked_model_tests", "attention_backward_model_tests",
    "cross_attention_model_tests", "cross_attention_masked_model_tests", "cross_attention_backward_model_tests",
    # the models around it
    "elm_model_tests", "local_encoder_smoke_test", "local_encoder_k_split", "local_decoder_k_split",
    "blt_model_generate_sanity", "model_stage_split_equivalence", "model_multi_doc_isolation",
    "model_decode_nullable_loss", "decoder_d0_modes",
    # KV cache: cached logits == dense logits, rollback / commit (tests/unit/infer/unit_kv_cache.c:158-336)
    "kv_cache_logits_equal_dense", "kv_cache_rollback_commit",
    # decisions: verify-draft cases A-D, BLT-S == greedy (tests/unit/infer/unit_self_speculation.c:178-255, :280-)
    "verify_draft_directed", "selfspec_structural_random", "selfspec_equivalence_trained",
    # block drafting, BLT-DV == greedy byte for byte (tests/unit/infer/unit_block_generation.c:499-554)
    "blockgen_draft_behavior", "blockgen_generation_gates", "blockgen_stage6_helpers",
    # block diffusion (tests/unit/models/unit_block_diffusion.c:186-238 and the training gates)
    "block_diffusion_gradcheck", "block_diffusion_overfit_gate", "block_diffusion_no_label_leak",
    "block_diffusion_last_row_upweight", "block_diffusion_draft_trailing_closed",
    # against the fixtures of the reference's PyTorch twin (tests/parity/*.c, tolerance 1e-4)
    "transformer_parity_tests", "local_encoder_parity", "global_transformer_parity", "local_decoder_parity",
    # training loops that must still converge with the new forward operator
    "elm_overfit_tests", "lencoder_overfit_test", "global_transformer_overfit", "local_decoder_overfit",
    "blt_model_overfit",
]
CUDA_TESTS = [
    "cuda_arena_transfer_tests",   # scaffolding sanity: the reference's own arena on this GPU
    "cuda_parity_composites",      # mask builders on the CUDA backend == CPU builders (parity_cuda_composites.c:48-160)
    "cuda_parity_training_step",   # decoder forward + backward, CUDA backend vs CPU backend (parity_cuda_model.c:133-372)
]


def _run(exe: Path, name: str, extra_env=None):
    if not exe.exists():
        pytest.skip(f"{exe.name} not built (make -C oracle accept REF=<reference tree>)")
    env = dict(os.environ)
    env["FBLT_REF_TEST_DATA"] = str(REF / "data" / "tests")
    env.update(extra_env or {})
    r = subprocess.run([str(exe), name], cwd=str(REF), env=env, capture_output=True, text=True, timeout=900)
    return r


@pytest.mark.parametrize("name", STAGE_TESTS)
def test_reference_test_on_staged_operator(cuda_lib, name):
    r = _run(STAGE, name, {"FBLT_STAGE_STRICT": "1"})
    assert r.returncode == 0 and f"[PASS] {name}" in r.stdout, (r.stdout[-2000:], r.stderr[-4000:])
    m = re.search(r"\[stage\] (\d+) operator calls on the GPU; .*; (\d+) outside tolerance", r.stderr)
    assert m, r.stderr[-2000:]
    assert int(m.group(1)) > 0, "the test never reached the GPU operator"
    assert int(m.group(2)) == 0


@pytest.mark.parametrize("name", CUDA_TESTS)
def test_reference_cuda_backend_test(cuda_lib, name):
    r = _run(CUDA, name, {"FBLT_REPORT_LAUNCHES": "1"})
    assert r.returncode == 0 and f"[PASS] {name}" in r.stdout, (r.stdout[-2000:], r.stderr[-4000:])
    m = re.search(r"\[fblt\] (\d+) kernel launches", r.stderr)
    assert m, r.stderr[-2000:]
    if name != "cuda_arena_transfer_tests":
        assert int(m.group(1)) > 0, "the reference's CUDA backend never reached the library"
