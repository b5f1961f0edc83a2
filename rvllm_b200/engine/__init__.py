from .batch import BatchBuilder, GroupContext, StepContext, StepEntry
from .loading import load_model, make_cache, parse_dtype
from .runner import ModelRunner
