"""Step function, scheduler and the user-facing engine.  Attributes are
imported on first use so that `engine.sequence` can be imported by the cache
package without pulling the whole engine in."""

_LAZY = {
    "LLMEngine": ".llm_engine", "RequestOutput": ".llm_engine", "StepOutput": ".llm_engine",
    "EngineStats": ".llm_engine", "ModelRunner": ".runner", "StepItem": ".runner",
    "Scheduler": ".scheduler", "SchedulerOutput": ".scheduler", "ScheduledSequence": ".scheduler",
    "Sequence": ".sequence", "SequenceStatus": ".sequence",
}


def __getattr__(name):
    if name in _LAZY:
        import importlib
        return getattr(importlib.import_module(_LAZY[name], __name__), name)
    raise AttributeError(name)
