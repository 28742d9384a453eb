"""connect6_b200 -- B200 (sm_100a) inference engine for the Connect6 policy/value CNN.

Drop-in for the inference hot path of mgxmateusz/connect6:
  model.PolicyValueNet / build_model / mask_logits      (connect6/model.py)
  history.HistoricalPolicyEnsemble                      (connect6/history.py:186-303)
  selfplay._sample_actions, D4 helpers, network input   (connect6/train.py:195-277,
                                                         connect6/vector_env.py:196-218)
Everything executes in hand-written CUDA behind the C ABI of include/c6_engine.h.
"""
from .engine import Engine
from .history import HistoricalCheckpoint, HistoricalPolicyEnsemble
from .model import PolicyValueNet, build_model, mask_logits

__all__ = ["Engine", "HistoricalCheckpoint", "HistoricalPolicyEnsemble", "PolicyValueNet", "build_model",
           "mask_logits"]
__version__ = "0.1.0"
