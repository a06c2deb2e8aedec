"""Public names of the package."""
from .config import (ConfigError, Qwen3Config, plan_from_config_json, register_architecture,  # noqa: F401
                     registered_architectures)
from .weights import WeightError, write_model_dir  # noqa: F401
from .cache import CacheManager, OutOfPages  # noqa: F401
from .engine import (AdmissionError, LLMEngine, ModelRunner, Scheduler, SchedulerConfig, StepEntry, StepError,  # noqa: F401
                     StepOutput, load_model_dir)
from .sampling import SamplingParams  # noqa: F401

__all__ = ["ConfigError", "Qwen3Config", "plan_from_config_json", "register_architecture",
           "registered_architectures", "WeightError", "write_model_dir", "CacheManager", "OutOfPages",
           "ModelRunner", "StepEntry", "StepError", "load_model_dir", "AdmissionError", "LLMEngine", "Scheduler",
           "SchedulerConfig", "StepOutput", "SamplingParams"]
