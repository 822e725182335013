from .grad_accumulation import accumulate_gradients
from .optimizer import Optimizer, create_lr_schedule, create_optimizer

__all__ = ["create_optimizer", "create_lr_schedule", "accumulate_gradients", "Optimizer"]
