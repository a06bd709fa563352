"""Module with the reference's import surface (``from moe import create_moe_layer``,
``models/mla_block.py:52-55``): put this package's directory ahead of the reference's ``models``
directory on ``sys.path`` under the name ``moe``, or assign the names below onto the reference's
``moe`` module before the model is built.  Both branches of the factory are provided."""
from .layer import (AuxLossFreeRouter, BatchedExperts, LatentBatchedExperts, LatentMoELayer, MoELayer,  # noqa: F401
                    SwiGLUExpert, create_moe_layer)
