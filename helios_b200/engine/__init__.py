from .batch import SeqSlice, StepContext, StepEntry, build_context

__all__ = ["SeqSlice", "StepContext", "StepEntry", "build_context"]
