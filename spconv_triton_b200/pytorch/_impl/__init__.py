"""Thin wrappers over libspconv_b200.so: the three private modules the
operator layer (``pytorch/ops.py``) is written against."""
