"""Plain, slow, whole-sequence implementation that the engine is measured against.

Nothing here imports the product package: it has its own config reading, its
own safetensors reading, its own formulas. It rests on the reference's
formulas (each function cites the reference file and line it was written
from); `tests/golden/` holds the one-off comparison of this implementation
with the reference's own numpy model code on tiny random models.
"""
