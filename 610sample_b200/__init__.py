"""B200 (sm_100a) attention forward / backward / double-backward kernels behind the
``attention_cuda`` + ``flash_attention_v7`` surface of JohnHeibel/610Sample.

The directory name is not a Python identifier; either put this directory on
``sys.path`` (then ``import attention_cuda`` and ``from attention import
flash_attention_v7`` work exactly as with the reference), or load it with
``importlib.import_module("610sample_b200")``.
"""
