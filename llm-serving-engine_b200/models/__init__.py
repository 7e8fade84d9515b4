from .decoder import DecoderModel
from .plan import CheckpointLayout, ModelPlan, ParamSource, RunEntry, Source

__all__ = ["DecoderModel", "CheckpointLayout", "ModelPlan", "ParamSource", "RunEntry", "Source"]
