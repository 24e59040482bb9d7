from .loader import TokenLoader, EnsembleTokenLoader
from .synthetic import write_synthetic_corpus, zipf_tokens
