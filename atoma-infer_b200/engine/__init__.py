from .engine import Engine, RequestMetrics, RequestOutput
from .runtime import LoadedModel, load_model, make_runtime
from .scheduler import PlannedEntry, Scheduler, StepPlan
from .step import StepEntry, StepFunction
