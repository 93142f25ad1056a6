"""Drop-in names of the reference's `flash_decoding` package: split-KV decode attention for
dense GQA caches (gqa) and MLA-style latent caches (mla, mla2)."""
from . import deepseek_mla, gqa, mla, mla2  # noqa: F401
