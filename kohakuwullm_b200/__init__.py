"""kohakuwullm_b200 — a B200-native (sm_100a) decoder-only LM pretraining framework.

Public surface: ``build(spec, REGISTRY)`` component construction, the pure
``LMBackbone(tokens, seq_info)`` trunk with a separate ``LMHead``, a DDP trainer with
token-exact gradient accumulation over packed varlen batches, the cost-measured pipeline engine
(``kohakuwullm_b200.pipe``) and portable whole-model-named checkpoints. The hot operations are
hand-written CUDA kernels for Blackwell (``kohakuwullm_b200/csrc``) bound through ctypes.
"""

__version__ = "0.1.0"
