"""B200-native (sm_100a) kernels for the PCVR token-mixing inference path, behind the operator
API of the TAAC_2026 experiment workspace.  See ``ops`` for the operator boundary, ``onetrans``
for the inference model and ``include/tb200.h`` for the C ABI."""

__version__ = "0.1.0"
