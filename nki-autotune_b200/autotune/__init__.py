"""B200-native stand-in for the ``autotune`` package of awslabs/nki-autotune.

Only the profiling path is provided: ``autotune.runner.api.profile`` with its
``KernelJob`` / ``ProfileResult`` / ``ProfileOutput`` types, backed by hand-written
sm_100a kernels reached through the C ABI of ``libb200_autotune.so``.
"""
