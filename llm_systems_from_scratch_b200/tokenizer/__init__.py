from .bpe import (PRE_TOKENIZE_REGEX, BPETokenizer, BPETokenizerParams, Tokenizer, find_chunk_boundaries,  # noqa: F401
                  get_chunk)
