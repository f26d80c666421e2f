"""Blackwell (sm_100a) build of Flint's GPT-2 training-step kernels.

``flint_b200.Flint`` loads ``flint_b200/lib/libflint.so`` (the C ABI declared in
``include/flint/flint.h`` plus the ``flint_b200_*`` extensions) and exposes the
same Python surface the reference's test bridge does.
"""

from .binding import (  # noqa: F401
    ERROR_CUDA,
    ERROR_INVALID_ARGUMENT,
    OK,
    Flint,
    FlintError,
    Gpt2,
    Gpt2Config,
    Gpt2ParameterInfo,
    library_path,
)
