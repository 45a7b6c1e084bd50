from .runner import GroupView, ModelRunner, StepContext, StepEntry, StepError

__all__ = ["GroupView", "ModelRunner", "StepContext", "StepEntry", "StepError"]
