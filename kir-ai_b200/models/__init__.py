"""Architectures as plans of parts; importing this package registers them."""
from .plan import DecoderModel, LayerCall, ModelPlan, PlanError

__all__ = ["DecoderModel", "LayerCall", "ModelPlan", "PlanError"]
