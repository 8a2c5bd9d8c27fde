"""Block-sparse linear layers of LeanTransformer on CUDA kernels.

Two weight orders are supported, as in the reference (lean_transformer/blocksparse/__init__.py): the
"native" order [in_features, blocks_per_input, block] for balanced layouts, and the "triton" order
[1, nnz, block, block] (blocks sorted like ``layout.nonzero()``) for layouts with uneven rows.  Both run
on the same kernels; they differ only in the index tables handed to them, and ``convert`` turns a weight stored in
one order into the other.
"""
from .layout import *  # noqa: F401,F403
from .layout import (butterfly_factor_to_matrix, get_blocksparse_layout, get_butterfly_layout,  # noqa: F401
                     get_hypercube_layout, get_indices_from_layout, register_blocksparse_layout)
from .linear import GeneralizedLinear, GeneralizedMatrix, _GeneralizedLinear  # noqa: F401
from .native_backend import blocksparse_matmul, blocksparse_matmul_backward  # noqa: F401
from .triton_backend import TRITON_PAD_TO, TritonMatmulForLinearLayer  # noqa: F401
from . import convert  # noqa: F401,E402
