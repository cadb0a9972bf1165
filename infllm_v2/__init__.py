"""Drop-in alias: `import infllm_v2` resolves to the B200 implementation, so existing call sites
of OpenBMB/infllmv2_cuda_impl (infllm_v2/__init__.py:3-11) keep working unchanged."""
from infllmv2_cuda_impl_b200 import *  # noqa: F401,F403
from infllmv2_cuda_impl_b200 import __all__, __version__  # noqa: F401
