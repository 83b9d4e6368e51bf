"""Data pipeline: memory-mapped indexed datasets, GPT / pairwise / online / synthetic datasets,
blending, distributed batch sampling and the C++ index builders."""
