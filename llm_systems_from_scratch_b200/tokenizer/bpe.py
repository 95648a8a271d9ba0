"""Byte-level BPE: training, encoding, decoding, file formats and CLI.

API and formats follow the reference (tokenizer/BPETokenizer.py:14-331): GPT-2 style pre-token regex;
ids are special tokens first, then the 256 bytes, then merges in creation order; ties between
equally frequent pairs go to the lexicographically greatest pair; ``vocab.json`` maps the
latin-1 decoding of each token's bytes to its id; ``merges.json`` is a list of
``[base64(left), base64(right)]``; encoded corpora are flat little-endian uint32 files.

The trainer is different: the reference recounts every pair and rewrites every word for each merge
(O(merges x corpus)).  Here pair counts are maintained incrementally - each merge only touches the
words that contain the merged pair, found through a pair -> words index - which produces the same
merges in the same order.  ``encode`` caches merged pre-tokens and prints no progress bar.
"""
from __future__ import annotations

import base64
import json
import mmap
import multiprocessing
import os
import re
import time
from collections import Counter, defaultdict
from dataclasses import dataclass
from functools import partial
from typing import BinaryIO, Iterable, Iterator, Optional

import regex

PRE_TOKENIZE_REGEX = r"'(?:[sdmt]|ll|ve|re)| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"
_PRE = regex.compile(PRE_TOKENIZE_REGEX)


def find_chunk_boundaries(file: BinaryIO, desired_num_chunks: int, split_special_token: bytes) -> list[int]:
    """Byte offsets that cut ``file`` into at most ``desired_num_chunks`` pieces without splitting a document: the
    file is mapped into memory and every interior cut is moved forward to the next occurrence of
    ``split_special_token`` with one ``find`` (to the end of the file when there is none).  Same contract as the
    reference helper (tokenizer/BPETokenizer.py:14-49): sorted, de-duplicated, first 0 and last the file size."""
    if not isinstance(split_special_token, bytes):
        raise TypeError("Must represent special token as a bytestring")
    size = os.fstat(file.fileno()).st_size
    if size == 0:
        return [0]
    with mmap.mmap(file.fileno(), 0, access=mmap.ACCESS_READ) as view:
        interior = (view.find(split_special_token, k * (size // desired_num_chunks)) for k in range(1, desired_num_chunks))
        cuts = {0, size} | {size if hit < 0 else hit for hit in interior}
    return sorted(cuts)


def get_chunk(input_path: str, desired_num_chunks: int) -> list[str]:
    """The pieces of ``input_path`` between the boundaries of ``find_chunk_boundaries``, decoded as UTF-8."""
    with open(input_path, "rb") as f:
        cuts = find_chunk_boundaries(f, desired_num_chunks, b"<|endoftext|>")
        if len(cuts) < 2:
            return []
        with mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ) as view:
            return [view[a:b].decode("utf-8", errors="ignore") for a, b in zip(cuts, cuts[1:])]


@dataclass
class BPETokenizerParams:
    vocab: dict[int, bytes]
    merges: list[tuple[bytes, bytes]]


def _count_chunk(text: str, special_tokens: list[str]) -> Counter:
    """Pre-token frequencies of one chunk; text is split on the special tokens first."""
    pieces = re.split("|".join(re.escape(t) for t in special_tokens), text) if special_tokens else [text]
    freqs: Counter = Counter()
    for piece in pieces:
        for m in _PRE.finditer(piece):
            freqs[tuple(bytes([b]) for b in m.group().encode("utf-8"))] += 1
    return freqs


class BPETokenizer:
    """Trainer.  ``train`` -> (vocab, merges); ``save`` writes the two JSON files."""

    def __init__(self, params: Optional[BPETokenizerParams] = None) -> None:
        self.vocab: dict[int, bytes] = params.vocab if params else {}
        self.merges: list[tuple[bytes, bytes]] = params.merges if params else []

    def pre_tokenize(self, text: str) -> Counter:
        return _count_chunk(text, [])

    @staticmethod
    def _pre_tokenize_chunk(text: str, special_tokens: list[str]) -> Counter:
        return _count_chunk(text, special_tokens)

    def train(self, input_path: str, vocab_size: int, special_tokens: list[str], num_workers: int | None = None,
              verbose: bool = True):
        log = print if verbose else (lambda *a, **k: None)
        t0 = time.time()
        log(f"[Train] input={input_path}, target_vocab_size={vocab_size}, special_tokens={special_tokens}")
        self.vocab = {i: tok.encode("utf-8") for i, tok in enumerate(special_tokens)}
        base = len(special_tokens)
        for b in range(256):
            self.vocab[base + b] = bytes([b])
        self.merges = []
        workers = num_workers or multiprocessing.cpu_count()
        chunks = get_chunk(input_path, workers)
        log(f"[Train] Chunked into {len(chunks)} parts")
        fn = partial(_count_chunk, special_tokens=special_tokens)
        if len(chunks) > 1 and workers > 1:
            with multiprocessing.Pool(min(workers, len(chunks))) as pool:
                counters = pool.map(fn, chunks)
        else:
            counters = [fn(c) for c in chunks]
        freqs: Counter = Counter()
        for c in counters:
            freqs.update(c)
        log(f"[Train] Pre-tokenized {len(freqs)} unique sequences ({time.time() - t0:.2f}s)")

        words = [list(w) for w in freqs]
        counts = [freqs[w] for w in freqs]
        pair_count: dict[tuple[bytes, bytes], int] = defaultdict(int)
        where: dict[tuple[bytes, bytes], set[int]] = defaultdict(set)
        for wi, w in enumerate(words):
            for a, b in zip(w, w[1:]):
                pair_count[(a, b)] += counts[wi]
                where[(a, b)].add(wi)
        t1 = time.time()
        next_id = len(self.vocab)
        while len(self.vocab) < vocab_size:
            live = [(c, p) for p, c in pair_count.items() if c > 0]
            if not live:
                log(f"[Train] No pairs left, stopped at vocab_size={len(self.vocab)}")
                break
            _, (left, right) = max(live)
            merged = left + right
            for wi in list(where[(left, right)]):
                w, c = words[wi], counts[wi]
                for a, b in zip(w, w[1:]):              # retire this word's old pairs
                    pair_count[(a, b)] -= c
                    where[(a, b)].discard(wi)
                new, i = [], 0
                while i < len(w):
                    if i + 1 < len(w) and w[i] == left and w[i + 1] == right:
                        new.append(merged)
                        i += 2
                    else:
                        new.append(w[i])
                        i += 1
                words[wi] = new
                for a, b in zip(new, new[1:]):          # and count its new ones
                    pair_count[(a, b)] += c
                    where[(a, b)].add(wi)
            pair_count.pop((left, right), None)
            where.pop((left, right), None)
            self.vocab[next_id] = merged
            self.merges.append((left, right))
            next_id += 1
        log(f"[Train] Merging done ({time.time() - t1:.2f}s)")
        log(f"[Train] Complete in {time.time() - t0:.2f}s — vocab_size={len(self.vocab)}, merges={len(self.merges)}")
        return self.vocab, self.merges

    def save(self, vocab_filepath: str, merges_filepath: str) -> None:
        with open(vocab_filepath, "w") as f:
            json.dump({tok.decode("latin1"): i for i, tok in self.vocab.items()}, f, ensure_ascii=False)
        with open(merges_filepath, "w") as f:
            json.dump([[base64.b64encode(a).decode("ascii"), base64.b64encode(b).decode("ascii")]
                       for a, b in self.merges], f)

    def get_params(self) -> BPETokenizerParams:
        return BPETokenizerParams(vocab=self.vocab, merges=self.merges)


class Tokenizer:
    """Encoder / decoder for a trained vocabulary."""

    def __init__(self, vocab: dict[int, bytes], merges: list[tuple[bytes, bytes]],
                 special_tokens: list[str] | None = None):
        self.id_to_bytes = dict(vocab)
        self.merges = merges
        self.special_tokens = special_tokens or []
        self.bytes_to_id = {tok: i for i, tok in self.id_to_bytes.items()}
        self.special_tokens_bytes = [s.encode("utf-8") for s in self.special_tokens]
        self.special_tokens_set = set(self.special_tokens_bytes)
        for tok in self.special_tokens_bytes:      # unknown specials are appended after the vocabulary
            if tok not in self.bytes_to_id:
                new_id = len(self.id_to_bytes)
                self.id_to_bytes[new_id] = tok
                self.bytes_to_id[tok] = new_id
        self.merge_ranks = {pair: rank for rank, pair in enumerate(self.merges)}
        ordered = sorted(self.special_tokens, key=len, reverse=True)   # longest special wins
        self._split = re.compile("(" + "|".join(re.escape(t) for t in ordered) + ")") if ordered else None
        self._cache: dict[bytes, list[int]] = {}

    @classmethod
    def from_files(cls, vocab_filepath: str, merges_filepath: str, special_tokens: list[str] | None = None):
        with open(vocab_filepath, "r") as f:
            vocab = {int(i): bytes(tok, "latin1") for tok, i in json.load(f).items()}
        with open(merges_filepath, "r") as f:
            merges = [(base64.b64decode(a), base64.b64decode(b)) for a, b in json.load(f)]
        return cls(vocab, merges, special_tokens)

    def _pre_tokenize(self, text: str) -> list[str]:
        return _PRE.findall(text)

    def _apply_merges(self, token: bytes) -> list[bytes]:
        """Repeatedly merge the adjacent pair with the lowest merge rank."""
        word = [bytes([b]) for b in token]
        while len(word) > 1:
            best_rank, best = None, None
            for pair in zip(word, word[1:]):
                rank = self.merge_ranks.get(pair)
                if rank is not None and (best_rank is None or rank < best_rank):
                    best_rank, best = rank, pair
            if best is None:
                break
            out, i = [], 0
            while i < len(word):
                if i + 1 < len(word) and word[i] == best[0] and word[i + 1] == best[1]:
                    out.append(best[0] + best[1])
                    i += 2
                else:
                    out.append(word[i])
                    i += 1
            word = out
        return word

    def _encode_pretoken(self, raw: bytes) -> list[int]:
        ids = self._cache.get(raw)
        if ids is None:
            ids = [self.bytes_to_id[part] for part in self._apply_merges(raw)]
            if len(self._cache) < 1_000_000:
                self._cache[raw] = ids
        return ids

    def encode(self, text: str) -> list[int]:
        out: list[int] = []
        for segment in (self._split.split(text) if self._split else [text]):
            if not segment:
                continue
            raw = segment.encode("utf-8")
            if raw in self.special_tokens_set:
                out.append(self.bytes_to_id[raw])
                continue
            for tok in _PRE.findall(segment):
                out.extend(self._encode_pretoken(tok.encode("utf-8")))
        return out

    def encode_iterable(self, iterable: Iterable[str]) -> Iterator[int]:
        for line in iterable:
            yield from self.encode(line)

    def decode(self, ids: list[int]) -> str:
        return b"".join(self.id_to_bytes[i] for i in ids).decode("utf-8", errors="replace")


def main(argv=None):
    import argparse

    import numpy as np
    ap = argparse.ArgumentParser(description="Train or encode with a BPE tokenizer")
    sub = ap.add_subparsers(dest="command", required=True)
    tr = sub.add_parser("train", help="Train a BPE tokenizer")
    tr.add_argument("--input", type=str, required=True)
    tr.add_argument("--vocab-size", type=int, required=True)
    tr.add_argument("--special-tokens", type=str, nargs="*", default=["<|endoftext|>"])
    tr.add_argument("--vocab-output", type=str, default="vocab.json")
    tr.add_argument("--merges-output", type=str, default="merges.txt")
    en = sub.add_parser("encode", help="Encode a text file into a uint32 token file")
    en.add_argument("--input", type=str, required=True)
    en.add_argument("--vocab", type=str, required=True)
    en.add_argument("--merges", type=str, required=True)
    en.add_argument("--special-tokens", type=str, nargs="*", default=["<|endoftext|>"])
    en.add_argument("--output", type=str, required=True)
    args = ap.parse_args(argv)
    if args.command == "train":
        t = BPETokenizer()
        t.train(args.input, args.vocab_size, args.special_tokens)
        t.save(args.vocab_output, args.merges_output)
        print(f"[Train] Saved vocab ({len(t.vocab)} tokens) -> {args.vocab_output}")
        print(f"[Train] Saved merges ({len(t.merges)} merges) -> {args.merges_output}")
    else:
        tok = Tokenizer.from_files(args.vocab, args.merges, args.special_tokens)
        print(f"[Encode] Loaded tokenizer (vocab={args.vocab}, merges={args.merges})")
        with open(args.input, "r", encoding="utf-8") as f:
            text = f.read()
        print(f"[Encode] Read {len(text)} characters from {args.input}")
        t0 = time.time()
        ids = tok.encode(text)
        print(f"[Encode] Encoded {len(ids)} tokens ({time.time() - t0:.2f}s)")
        np.array(ids, dtype=np.uint32).tofile(args.output)
        print(f"[Encode] Saved uint32 array -> {args.output}")
        print(f"[Encode] Load with: np.memmap('{args.output}', dtype=np.uint32, mode='r')")


if __name__ == "__main__":
    main()
