from .context import StepContext, Workspace
from .engine import Engine, StepError
from .generate import Generated, GenerationError, Request, generate, plan_batches, run_batch, tokens_reserved
from .model import DecoderModel, parse_dtype

__all__ = ["DecoderModel", "Engine", "Generated", "GenerationError", "Request", "StepContext", "StepError",
           "Workspace", "generate", "parse_dtype", "plan_batches", "run_batch", "tokens_reserved"]
