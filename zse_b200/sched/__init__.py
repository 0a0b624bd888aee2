from .batch_runner import BatchRunner, StepResult
from .draft_model import NGramDraftModel, SelfDraftModel
from .memory_budget import MemoryBudget
from .queue import RequestQueue
from .request import FinishReason, GenerationParams, InferenceRequest, RequestOutput, RequestState
from .sampler import Sampler
from .scheduler import Scheduler, SchedulerConfig, SchedulerOutput, StepType
from .spec_runner import SpeculativeRunner
from .verifier import SpeculativeVerifier, VerifyResult
