"""Kernel backends. ``ternary_b200`` sits where the reference keeps ``ternary_cuda.py``, ``cpu.py`` and ``torch_ref.py``."""
