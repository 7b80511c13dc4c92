from .sequence import Sequence, SequenceStatus
from .scheduler import Scheduler
from .model_runner import ModelRunner, StepItem
from .llm_engine import LLMEngine
