"""Train a byte-level BPE tokenizer on a sample of Parquet corpora, keeping only text of one script.

    python tokenizer_train.py --data-path data/da:0.05 --data-path data/en:0.01 --output tok.json
           [--text-column text] [--vocab-size 50000] [--script latin] [--max-other-ratio 0.1]
           [--batch-size 1000] [--seed 42] [--extra-special "<|im_start|>,<|im_end|>"]

Each ``--data-path DIR:RATE`` contributes a Bernoulli(RATE) sample of its rows (drawn per row group so
only sampled groups are read).  A text is kept when at most ``max-other-ratio`` of its letters
belong to scripts other than the chosen one (digits, punctuation and whitespace are neutral).
Tokenizer: ByteLevel pre-tokenizer (prefix space) / decoder / post-processor, special tokens
``<bos>``, ``<eos>`` first (reference: tokenizer_train.py:21-76 script filter, :78-195 sampler,
:209-320 trainer).
"""
from __future__ import annotations

import argparse
import random
import unicodedata
from pathlib import Path
from typing import Iterator

SCRIPT_PRESETS = {
    "latin": ("LATIN",), "cyrillic": ("CYRILLIC",), "arabic": ("ARABIC",), "devanagari": ("DEVANAGARI",),
    "chinese": ("CJK",), "greek": ("GREEK",), "hebrew": ("HEBREW",), "any": (),
}


class ScriptFilter:
    """Keeps text whose letters are (almost) all of one Unicode script; script = first word(s) of the
    character name, cached per code point."""

    def __init__(self, prefixes: tuple[str, ...], max_other_ratio: float = 0.1):
        self.prefixes, self.max_other_ratio = prefixes, max_other_ratio
        self._cache: dict[str, bool] = {}

    @classmethod
    def from_preset(cls, script: str, max_other_ratio: float = 0.1) -> "ScriptFilter":
        if script not in SCRIPT_PRESETS:
            raise ValueError(f"unknown script {script!r}; choose from {sorted(SCRIPT_PRESETS)}")
        return cls(SCRIPT_PRESETS[script], max_other_ratio)

    def _in_script(self, ch: str) -> bool:
        hit = self._cache.get(ch)
        if hit is None:
            hit = unicodedata.name(ch, "").startswith(self.prefixes)
            self._cache[ch] = hit
        return hit

    def should_keep_text(self, text: str) -> bool:
        if not self.prefixes:
            return bool(text)
        letters = other = 0
        for ch in text:
            if ch.isalpha():
                letters += 1
                if not self._in_script(ch):
                    other += 1
        return letters > 0 and other <= self.max_other_ratio * letters


class ParquetSampler:
    """Bernoulli row sample over several directories, read row group by row group."""

    def __init__(self, sources: list[tuple[Path, float]], text_column: str = "text", seed: int = 42,
                 text_filter: ScriptFilter | None = None):
        self.sources, self.text_column, self.seed, self.filter = sources, text_column, seed, text_filter
        self.seen = self.kept = 0

    @staticmethod
    def parse(spec: str) -> tuple[Path, float]:
        path, _, rate = spec.rpartition(":")
        if not path:
            return Path(rate), 1.0
        return Path(path), float(rate)

    def files(self) -> list[tuple[Path, float]]:
        out = []
        for root, rate in self.sources:
            found = [root] if root.is_file() else sorted(root.rglob("*.parquet"))
            if not found:
                raise FileNotFoundError(f"no parquet files under {root}")
            out.extend((f, rate) for f in found)
        return out

    def sample_iterator(self, batch_size: int = 1000) -> Iterator[list[str]]:
        import pyarrow.parquet as pq
        rng = random.Random(self.seed)
        batch: list[str] = []
        for path, rate in self.files():
            pf = pq.ParquetFile(path)
            for g in range(pf.metadata.num_row_groups):
                n = pf.metadata.row_group(g).num_rows
                picks = [i for i in range(n) if rng.random() < rate]
                if not picks:
                    continue
                col = pf.read_row_group(g, columns=[self.text_column]).column(0)
                for i in picks:
                    text = col[i].as_py()
                    self.seen += 1
                    if isinstance(text, str) and (self.filter is None or self.filter.should_keep_text(text)):
                        self.kept += 1
                        batch.append(text)
                        if len(batch) == batch_size:
                            yield batch
                            batch = []
        if batch:
            yield batch


def train_tokenizer(batches: Iterator[list[str]], vocab_size: int, extra_special: list[str] | None = None):
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, processors, trainers

    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=True)
    tok.decoder = decoders.ByteLevel()
    tok.post_processor = processors.ByteLevel(trim_offsets=True)
    trainer = trainers.BpeTrainer(vocab_size=vocab_size, special_tokens=["<bos>", "<eos>", *(extra_special or [])],
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False)
    tok.train_from_iterator(batches, trainer=trainer)
    return tok


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description="Train a byte-level BPE tokenizer on sampled Parquet text")
    ap.add_argument("--data-path", action="append", required=True, metavar="DIR:RATE")
    ap.add_argument("--text-column", default="text")
    ap.add_argument("--output", required=True)
    ap.add_argument("--vocab-size", type=int, default=50000)
    ap.add_argument("--script", default="latin", choices=sorted(SCRIPT_PRESETS))
    ap.add_argument("--batch-size", type=int, default=1000)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--max-other-ratio", type=float, default=0.1)
    ap.add_argument("--extra-special", default="", help="comma-separated additional special tokens")
    a = ap.parse_args(argv)
    sampler = ParquetSampler([ParquetSampler.parse(s) for s in a.data_path], a.text_column, a.seed,
                             ScriptFilter.from_preset(a.script, a.max_other_ratio))
    tok = train_tokenizer(sampler.sample_iterator(a.batch_size), a.vocab_size, [t for t in a.extra_special.split(",") if t])
    out = Path(a.output)
    out.parent.mkdir(parents=True, exist_ok=True)
    tok.save(str(out))
    print(f"sampled {sampler.seen} texts, kept {sampler.kept}; vocabulary {tok.get_vocab_size()} -> {out}")


if __name__ == "__main__":
    main()
