from .causal_lm import CausalLM
from .plan import ExecStep, ModelPlan
from .registry import register_architecture, resolve, supported_architectures

__all__ = ["CausalLM", "ExecStep", "ModelPlan", "register_architecture", "resolve", "supported_architectures"]
