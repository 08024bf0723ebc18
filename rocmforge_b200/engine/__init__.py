from .batch import StepRequest, StepBatch, BatchError
from .context import Options, StepContext
from .stream import ResidualStream
from .model import Model, ModelSpec, ScheduleEntry
