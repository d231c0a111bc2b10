"""Checkpoint I/O in the V-MoE formats (single msgpack file and sharded .index/.data files)."""
from vmoe_b200.checkpoints.base import (find_latest_complete_checkpoint_for_prefix,
                                        iterate_complete_steps_for_prefix, remove_checkpoints,
                                        restore_checkpoint, restore_multiple_checkpoints,
                                        save_checkpoint, save_checkpoint_async,
                                        save_multiple_checkpoints_async)
from vmoe_b200.checkpoints.partitioned import ArraySharding, Version
from vmoe_b200.checkpoints.partitioned import restore_checkpoint as restore_checkpoint_partitioned
from vmoe_b200.checkpoints.partitioned import save_checkpoint as save_checkpoint_partitioned
