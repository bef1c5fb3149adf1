"""B200-native (sm_100a) Conv2d / ConvTranspose2d / Linear contraction path.

``nectarml_b200.ops``        tensor-level calls into the C ABI (``include/nectarml_b200.h``)
``nectarml_b200._nectarml``  drop-in for the reference's ``_nectarml.tensor.conv.*`` /
                             ``_nectarml.tensor.matmul`` host-op names
``nectarml_b200.build``      nvcc build of the shared library
"""
__all__ = ["ops", "build"]
