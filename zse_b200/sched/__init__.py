from .batch_runner import BatchRunner, StepResult
from .draft_model import NGramDraftModel, SelfDraftModel
from .memory_budget import MemoryBudget
from .queue import RequestQueue
from .request import FinishReason, GenerationParams, InferenceRequest, RequestOutput, RequestState
from .sampler import Sampler
from .scheduler import Scheduler, SchedulerConfig, SchedulerOutput, StepType
from .spec_runner import SpeculativeRunner
from .verifier import SpeculativeVerifier, VerifyResult


def __getattr__(name):
    """``ZStreamerEngine`` lives in ``zse_b200.engine`` (it owns the model as well as the scheduler); the reference exports
    it from its scheduling package, so it is reachable here too, loaded on first use."""
    if name == "ZStreamerEngine":
        from ..engine import ZStreamerEngine
        return ZStreamerEngine
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
