"""Registry of public corpora: fetch (when the machine has network access), extract, tokenise
(tools/datasets/corpora.py:35-380).  The registry is a table; one ``Corpus`` class does the work.

Files already present under ``<data_dir>/<name>/`` are never fetched again, so an air-gapped machine can be
fed by copying the archives there first; a missing file without network is a clear error, not a hang.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import tarfile
import urllib.request
import zipfile
from dataclasses import dataclass, field
from multiprocessing import cpu_count
from typing import List, Optional

GPT2_VOCAB_URL = "https://s3.amazonaws.com/models.huggingface.co/bert/gpt2-vocab.json"
GPT2_MERGE_URL = "https://s3.amazonaws.com/models.huggingface.co/bert/gpt2-merges.txt"
_EYE = "https://the-eye.eu/public/AI/pile_preliminary_components/"


@dataclass
class Corpus:
    name: str
    urls: List[str]
    num_docs: Optional[int] = None
    ftfy: bool = False
    tokenizer_type: str = "GPT2BPETokenizer"
    merge_file: Optional[str] = None
    vocab_file: Optional[str] = None
    data_dir: Optional[str] = None
    force_redownload: bool = False
    num_workers: Optional[int] = None
    _files: List[str] = field(default_factory=list)

    def configure(self, tokenizer_type=None, merge_file=None, vocab_file=None, data_dir=None,
                  force_redownload=None, num_workers=None):
        self.tokenizer_type = tokenizer_type or "GPT2BPETokenizer"
        self.data_dir = data_dir or os.environ.get("DATA_DIR", "./data")
        self.merge_file = merge_file or f"{self.data_dir}/gpt2-merges.txt"
        self.force_redownload = bool(force_redownload)
        if vocab_file is None:
            vocab_file = {"GPT2BPETokenizer": f"{self.data_dir}/gpt2-vocab.json", "HFGPT2Tokenizer": "gpt2",
                          "CharLevelTokenizer": None}.get(self.tokenizer_type, "MISSING")
            if vocab_file == "MISSING":
                raise AssertionError("vocab_file must be specified for this tokenizer type")
        self.vocab_file = vocab_file
        self.num_workers = num_workers or cpu_count()
        return self

    @property
    def base_dir(self):
        return os.path.join(self.data_dir, self.name)

    def exists(self):
        """A tokenised ``.bin`` is already there."""
        return os.path.isfile(os.path.join(self.base_dir, f"{self.name}_text_document.bin"))

    def download(self):
        os.makedirs(self.base_dir, exist_ok=True)
        for url in self.urls:
            dst = os.path.join(self.base_dir, os.path.basename(url))
            if os.path.isfile(dst) and not self.force_redownload:
                continue
            try:
                with urllib.request.urlopen(url, timeout=30) as r, open(dst + ".part", "wb") as f:
                    shutil.copyfileobj(r, f)
                os.replace(dst + ".part", dst)
            except Exception as e:  # noqa: BLE001
                raise RuntimeError(f"could not fetch {url} ({e}); copy the file to {dst} and run again") from e

    def extract(self) -> List[str]:
        """Unpack archives; returns the list of text files to tokenise."""
        out = []
        for url in self.urls:
            path = os.path.join(self.base_dir, os.path.basename(url))
            if path.endswith(".zip"):
                with zipfile.ZipFile(path) as z:
                    z.extractall(self.base_dir)
                    out += [os.path.join(self.base_dir, n) for n in z.namelist() if not n.endswith("/")]
            elif path.endswith((".tar", ".tar.gz", ".tgz")):
                with tarfile.open(path) as t:
                    t.extractall(self.base_dir, filter="data")
                    out += [os.path.join(self.base_dir, m.name) for m in t.getmembers() if m.isfile()]
            else:
                out.append(path)
        return out

    def tokenize(self, files: List[str]):
        from . import preprocess_data
        argv = ["--input", ",".join(files), "--output-prefix", os.path.join(self.base_dir, self.name),
                "--tokenizer-type", self.tokenizer_type, "--dataset-impl", "mmap", "--append-eod",
                "--workers", str(self.num_workers)]
        if self.vocab_file:
            argv += ["--vocab-file", self.vocab_file]
        if self.merge_file and self.tokenizer_type == "GPT2BPETokenizer":
            argv += ["--merge-file", self.merge_file]
        if self.num_docs is not None:
            argv += ["--num-docs", str(self.num_docs)]
        if self.ftfy:
            argv += ["--ftfy"]
        return preprocess_data.main(argv)

    def prepare(self):
        if self.exists() and not self.force_redownload:
            return
        self.download()
        self.tokenize(self.extract())


def _registry():
    pile = [f"https://the-eye.eu/public/AI/pile/train/{i:02}.jsonl.zst" for i in range(30)]
    return {
        "enron": Corpus("enron", ["http://eaidata.bmk.sh/data/enron_emails.jsonl.zst"], 517401),
        "pile_subset": Corpus("pile_00", pile[:1]),
        "pile": Corpus("pile", pile),
        "github": Corpus("github", ["http://eaidata.bmk.sh/data/github_small.jsonl.zst"]),
        "arxiv": Corpus("arxiv", [_EYE + "2020-09-08-arxiv-extracts-nofallback-until-2007-068.tar.gz"]),
        "europarl": Corpus("europarl", [_EYE + "EuroParliamentProceedings_1996_2011.jsonl.zst"]),
        "freelaw": Corpus("freelaw", [_EYE + "FreeLaw_Opinions.jsonl.zst"]),
        "nih": Corpus("nih", [_EYE + "NIH_ExPORTER_awarded_grant_text.jsonl.zst"]),
        "pubmed": Corpus("pubmed", [_EYE + "PMC_extracts.tar.gz"]),
        "books1": Corpus("books1", [_EYE + "books1.tar.gz"]),
        "books3": Corpus("books3", [_EYE + "books3.tar.gz"]),
        "hackernews": Corpus("hackernews", [_EYE + "hn.tar.gz"], 373000),
        "openwebtext2": Corpus("openwebtext2", ["https://huggingface.co/datasets/segyges/OpenWebText2/resolve/main/"
                                                "openwebtext2.jsonl.zst.tar"], 17103000),
        "stackexchange": Corpus("stackexchange", [_EYE + "stackexchange_dataset.tar"]),
        "ubuntu_irc": Corpus("ubuntu_irc", [_EYE + "ubuntu_irc_until_2020_9_1.jsonl.zst"]),
        "youtube_subtitles": Corpus("youtube_subtitles", [_EYE + "yt_subs.jsonl.zst"]),
        "c4": Corpus("c4", [f"https://the-eye.eu/eleuther_staging/c4/en/c4-train.{i:05}-of-01024.json.gz"
                            for i in range(1024)]),
        "c4_openwebtext": Corpus("c4_openwebtext", [f"https://the-eye.eu/eleuther_staging/c4/realnewslike/"
                                                    f"c4-train.{i:05}-of-00512.json.gz" for i in range(512)]),
        "enwik8": Corpus("enwik8", ["http://mattmahoney.net/dc/enwik8.zip"]),
    }


DATA_DOWNLOADERS = {"pass": "pass", **_registry()}


def maybe_download_gpt2_tokenizer_data(tokenizer_type, data_dir):
    if tokenizer_type not in (None, "GPT2BPETokenizer"):
        return
    for url, name in ((GPT2_VOCAB_URL, "gpt2-vocab.json"), (GPT2_MERGE_URL, "gpt2-merges.txt")):
        dst = os.path.join(data_dir, name)
        if not os.path.isfile(dst):
            try:
                urllib.request.urlretrieve(url, dst)
            except Exception as e:  # noqa: BLE001
                raise RuntimeError(f"could not fetch {url} ({e}); copy it to {dst}") from e


def prepare_dataset(dataset_name: str, tokenizer_type: str = None, data_dir: str = None, vocab_file: str = None,
                    merge_file: str = None, force_redownload: bool = None, num_workers: int = None):
    """Fetch + tokenise the registry entry ``dataset_name`` into ``data_dir``."""
    data_dir = data_dir or os.environ.get("DATA_DIR", "./data")
    os.makedirs(data_dir, exist_ok=True)
    entry = DATA_DOWNLOADERS.get(dataset_name.lower())
    if entry is None:
        raise NotImplementedError(f'Dataset "{dataset_name}" not recognized - please choose from '
                                  f'{list(DATA_DOWNLOADERS.keys())}')
    if entry == "pass":
        return
    maybe_download_gpt2_tokenizer_data(tokenizer_type, data_dir)
    entry.configure(tokenizer_type=tokenizer_type, vocab_file=vocab_file, merge_file=merge_file, data_dir=data_dir,
                    force_redownload=force_redownload, num_workers=1 if dataset_name == "enwik8" else num_workers)
    entry.prepare()
