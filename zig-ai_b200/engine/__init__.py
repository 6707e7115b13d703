"""The step function, the scheduler above it, generation and trace replay."""
from .batch import StepBatch, pack_step
from .runner import ModelRunner, StepError, load_runner, parse_dtype
from .scheduler import Request, RequestRefused, Scheduler, StepPlan
from .engine import Engine, generate
