"""CPU oracle for the Winograd convolution path.  TEST INFRASTRUCTURE, not the product.

Only the test-suite, ``__graft_entry__.smoke()`` and the CPU-baseline leg of ``bench.py`` may import
this package.  It restates the reference's numpy ground truth (``Conv_NCHW`` / ``Conv_NHWC`` /
``Conv_CHWN`` and the stage-by-stage ``Wino_*`` chain of ``layoutTest/*/data/WinoTran_*.py``) and is
pinned to outputs of those functions stored under ``tests/golden/``.
"""
from .direct import (conv_f64, conv_f32, conv_f32_plain, maxpool2x2, num_threads, set_num_threads, build,  # noqa: F401
                     LAYOUTS, to_layout, from_layout, filter_to_layout)
from .wino_stages import (matrices, tiles_per_side, input_transform, filter_transform,  # noqa: F401
                          tile_gemm, output_transform, winograd_conv, round_to)
