
from .pipeline import ContinuousBatchingPipeline, GenerationConfig, GenerationResult   # noqa: F401,E402
from .scheduler import SchedulerConfig   # noqa: F401,E402
from .llm_pipeline import ByteTokenizer, LLMPipeline   # noqa: F401,E402
