"""``tokenizer.BPETokenizer`` of the reference (tokenizer/BPETokenizer.py): same names, same files, same CLI."""
from llm_systems_from_scratch_b200.tokenizer.bpe import (  # noqa: F401
    PRE_TOKENIZE_REGEX, BPETokenizer, BPETokenizerParams, Tokenizer, find_chunk_boundaries, get_chunk, main)

if __name__ == "__main__":
    main()
