"""B200-native GDPA (Generalized Dot Product Attention) kernels behind the reference library's
``gdpa`` Python entry point.  Importing ``ads_model_kernel_library_b200.gdpa`` loads the C-ABI
kernel library ``libgdpa_b200.so`` (build it with ``python -m ads_model_kernel_library_b200.build``)."""

__version__ = "0.1.0"
