"""CPU oracle for the Monarch-Muon optimizer step.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory; it exists so the CUDA path can be checked against an independent
CPU restatement of the reference algorithm.  Only the test-suite, the smoke
entry and the benchmark's CPU-baseline / reference arm may import it.

Modules
-------
muon_oracle   heavy-ball momentum, batched quintic Newton-Schulz, the Muon
              weight update and the embedded AdamW, restated from
              pretrain/src/models/monarch/monarch_muon.py and its bf16 twin
              membench/src/models/monarch/monarch_muon.py.
fp8_oracle    the two FP8 (E4M3, groups of 128) optimizer-state codecs:
              plain absmax (pretrain/third_party/coat/optimizer/
              triton_kernels.py:34-36,51-63) and COAT dynamic-range expansion
              (pretrain/src/models/monarch/coat_state_muon.py:22-91); the
              momentum and AdamW steps on states held in those formats.
sft_oracle    the fine-tuning optimizer on fp32 master weights
              (finetune/sft_optimizer.py), pinned bit-exactly to the
              reference's own run.

make_ref      stages the reference project's own files, unmodified, under the
              git-ignored oracle/_ref/ (with a manifest of hashes).
ref_loader    imports those staged modules (the reference's Triton FP8 kernels,
              its optimizer classes, its training program) for the GPU parity
              tests and the benchmark's reference arms.

Parity pins.  (1) The restatement is checked in tests/test_oracle_golden.py
against vectors produced by importing and running the reference's own Python on
CPU (tests/golden/make_golden.py).  The expansion codec could not be executed on
CPU (its Triton kernel needs libdevice.pow), so fp8_oracle's restatement of that
codec has no CPU pin.  (2) On a GPU the reference itself is the arbiter:
tests/test_gpu_reference.py compares the CUDA kernels with the reference's
kernels and classes run from oracle/_ref/ - absmax codec bit for bit, expansion
codec to its measured residual.
"""
