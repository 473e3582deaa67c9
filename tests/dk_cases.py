"""Seeded synthetic inputs of the tests: the generators live in the package
(deformable_kernels/synthetic.py) because the bench and the golden-vector generator use them too."""
from deformable_kernels.synthetic import *  # noqa: F401,F403
from deformable_kernels.synthetic import _pair  # noqa: F401
