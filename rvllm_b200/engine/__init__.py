from .batch import BatchBuilder, GroupContext, StepContext, StepEntry
from .engine import Engine, RunResult, RunStats, run, settled_heap
from .generator import GenerateOptions, Generator, graphs_default
from .loading import load_model, make_cache, parse_dtype
from .runner import ModelRunner
from .scheduler import (FinishReason, Request, Scheduler, SchedulerConfig, SchedulerStats,
                        TokenEvent)
