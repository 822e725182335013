from .conversion import load_hf_checkpoint, save_hf_checkpoint
from .manager import (CheckpointManager, create_checkpoint_manager, maybe_restore_checkpoint, restore_checkpoint,
                      save_checkpoint, wait_for_checkpoint)

__all__ = ["CheckpointManager", "create_checkpoint_manager", "save_checkpoint", "restore_checkpoint",
           "maybe_restore_checkpoint", "wait_for_checkpoint", "load_hf_checkpoint", "save_hf_checkpoint"]
