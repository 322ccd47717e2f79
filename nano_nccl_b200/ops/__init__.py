"""Torch custom ops (``torch.ops.b200ccl.*``) over a registered communicator.

The ops take a communicator id instead of an object so that they can be traced and captured like
any other op. ``register_communicator`` returns the id; id 0 is the default communicator set by
``set_default_communicator``.
"""
from .collectives import (all_gather, all_reduce, all_reduce_, get_communicator, reduce_scatter,  # noqa: F401
                          register_communicator, set_default_communicator)
