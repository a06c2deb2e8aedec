"""The step function, the scheduler and the generation loop."""
from .loading import load_model_dir, parse_dtype, random_model  # noqa: F401
from .runner import ModelRunner, StepEntry, StepError  # noqa: F401
from .scheduler import AdmissionError, Scheduler, SchedulerConfig, Sequence  # noqa: F401
from .llm import LLMEngine, StepOutput  # noqa: F401
