"""deploy3d_b200: B200-native (sm_100a) sparse-convolution hot path behind deploy3d's plugin surface.

``deploy3d_b200.ops``      operator functions with the names/signatures of ``deploy3d.symfun.ops``
``deploy3d_b200.plugins``  plugin objects created from (name, data_s) like the reference's creators
``deploy3d_b200.build``    nvcc build of ``libs/libdeploy3d_b200.so`` (the C ABI in include/deploy3d_b200.h)
"""
__version__ = "0.1.0"
