"""Run-time policy of the engine, read once from the environment.

Mirrors ``upstride::Context`` (reference ``src/backend/backend.hpp:45-74``, ``src/backend/backend.cc:35-57``):
``UPSTRIDE_MEMORY_OPTIMIZED`` > 0 selects the 16-product formulation (default: the factorised 8-product
one), ``UPSTRIDE_CONV_FP16_POLICY`` in {"full16", "backward32"} selects the fp16 convolution policy
(anything else: fp32 compute), ``UPSTRIDE_VERBOSE`` enables logging.
"""
import enum
import os


class ConvFp16ComputePolicy(enum.IntEnum):
    FULL_32 = 0          # fp32 compute everywhere ("slow, accurate")
    FULL_16 = 1          # fp16 forward and backward ("fast, inaccurate")
    FORWARD_16_BACKWARD_32 = 2


def _int_env(name, default=0):
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


class Context:
    def __init__(self, environ=None):
        env = os.environ if environ is None else environ
        try:
            self.memory_optimized = int(env.get("UPSTRIDE_MEMORY_OPTIMIZED", 0)) > 0
        except ValueError:
            self.memory_optimized = False
        policy = env.get("UPSTRIDE_CONV_FP16_POLICY", "")
        if policy == "full16":
            self.conv_fp16_policy = ConvFp16ComputePolicy.FULL_16
        elif policy == "backward32":
            self.conv_fp16_policy = ConvFp16ComputePolicy.FORWARD_16_BACKWARD_32
        else:
            self.conv_fp16_policy = ConvFp16ComputePolicy.FULL_32
        try:
            self.verbose = int(env.get("UPSTRIDE_VERBOSE", 0)) > 0
        except ValueError:
            self.verbose = False

    def preferSpeedToMemory(self):
        """True selects the factorised 8-product formulation (reference ``backend.hpp:58``)."""
        return not self.memory_optimized

    def isFp16ConvForwardAllowed(self):
        return self.conv_fp16_policy in (ConvFp16ComputePolicy.FULL_16, ConvFp16ComputePolicy.FORWARD_16_BACKWARD_32)

    def isFp16ConvBackwardAllowed(self):
        return self.conv_fp16_policy == ConvFp16ComputePolicy.FULL_16

    def variant(self):
        from . import _lib
        return _lib.VARIANT_8_PRODUCT if self.preferSpeedToMemory() else _lib.VARIANT_16_PRODUCT
