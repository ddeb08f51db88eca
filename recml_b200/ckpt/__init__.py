"""Checkpointing: Orbax-layout directories, async manager, continuous-eval iterator."""
from recml_b200.ckpt.manager import (CheckpointManager, ShardedLeaf, all_steps,
                                     checkpoints_iterator, latest_step, restore_tree)
