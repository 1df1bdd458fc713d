"""B200-native Qwen2.5 Q4_0 inference hot path (sm_100a kernels behind a C-ABI, Python host).

The directory name starts with a digit, so import it with importlib:

    import importlib
    lab = importlib.import_module("3080lab_b200")
"""
