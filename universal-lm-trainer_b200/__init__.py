"""universal-lm-trainer_b200: the Universal-LM-Trainer training hot path on B200.

The directory name is not an importable identifier; put this directory on
``sys.path`` (as the reference's train.py does with its own directory,
train.py:79-82) and import the modules by name: ``flash_attn_v100_cuda``,
``flash_attn_v100``, ``ulm_ops``, ``ulm_model``, ``ulm_dp``.
"""
