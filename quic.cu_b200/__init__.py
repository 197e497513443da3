"""quic_b200 — the W4A16 decode token loop of hdahroug/quic.cu rebuilt for B200 (sm_100a).

The directory name contains a dot, so the package is imported under the name
``quic_cu_b200`` through ``__graft_entry__.load_package()`` at the repository root (or any
loader that registers this directory under that name).

Modules mirror the reference's layout: ``engine`` (src/engine.py), ``scheduler``
(src/scheduler.py), ``sequence`` (src/sequence.py), ``config`` (src/config.py), ``model``
(src/model.py), ``checkpoint`` (src/quant/checkpoint.py), ``kernels`` (kernels/__init__.py),
``replicas`` (one engine process per GPU; the reference is single-GPU).
Importing the package does not touch CUDA; the first kernel call loads the library.
"""

from .config import EngineConfig
from .scheduler import AdmissionDecision, BatchAdmissionPolicy, ContinuousAdmissionPolicy, StaticAdmissionPolicy
from .sequence import SequenceState

__all__ = [
    "EngineConfig", "AdmissionDecision", "BatchAdmissionPolicy", "ContinuousAdmissionPolicy",
    "StaticAdmissionPolicy", "SequenceState",
]
