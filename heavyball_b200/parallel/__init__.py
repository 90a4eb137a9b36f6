"""Distributed layer: sharded-parameter repartitioning (``fsdp``) and data-parallel gradient
reduction with owner-rank second-order work (``ddp``)."""
