from .loader import TokenLoader
from .synthetic import write_synthetic_corpus, zipf_tokens
