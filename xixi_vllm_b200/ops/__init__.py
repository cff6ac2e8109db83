"""Model ops.

* ``ops.cpu_ref``  - plain PyTorch: the oracle and the CPU/gloo backend.
* ``ops.cuda``     - ctypes bindings of the hand-written sm_100a kernels (``csrc/kernels``).
* ``ops.dispatch`` - what model code calls; routes on the tensor's device.
* ``ops.hostlib``  - host-side C++ helpers (hashing, batch metadata, safetensors reads).

Importing this package imports none of them (the CPU data plane must stay torch-free).
"""
