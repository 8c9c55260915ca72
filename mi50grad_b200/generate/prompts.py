"""Prompt set for measuring speculative-decoding acceptance.

Twenty prompts in four domains whose continuations repeat earlier text to
different degrees (code, JSON, conversation, deliberately repetitive text), a
60/40 splitter (the first part builds the n-gram cache, the rest is the
continuation to predict) and a tokenizer adapter with a character-level
fall-back so the tooling works without a model tokenizer.  Same role and class
names as the reference's dataset (src/inference/prompts.py:39-654,
data/test_prompts.json); the prompt texts are this project's own.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Dict, List, Optional, Tuple


class PromptCategory(str, Enum):
    CODE = "code"
    JSON = "json"
    CONVERSATIONAL = "conversational"
    REPETITIVE = "repetitive"


@dataclass
class Prompt:
    text: str
    category: PromptCategory
    description: str = ""
    expected_pattern: str = ""
    metadata: Dict[str, Any] = field(default_factory=dict)

    def to_dict(self) -> Dict[str, Any]:
        return {"text": self.text, "category": self.category.value, "description": self.description,
                "expected_pattern": self.expected_pattern, "metadata": dict(self.metadata)}

    @classmethod
    def from_dict(cls, data: Dict[str, Any]) -> "Prompt":
        return cls(text=data["text"], category=PromptCategory(data["category"]),
                   description=data.get("description", ""), expected_pattern=data.get("expected_pattern", ""),
                   metadata=dict(data.get("metadata", {})))


@dataclass
class TrainTestSplit:
    train_text: str
    test_text: str
    train_ids: List[int] = field(default_factory=list)
    test_ids: List[int] = field(default_factory=list)

    def __repr__(self) -> str:
        return (f"TrainTestSplit(train={len(self.train_ids) or len(self.train_text)}, "
                f"test={len(self.test_ids) or len(self.test_text)})")


def _code_prompts() -> List[Prompt]:
    P, C = Prompt, PromptCategory.CODE
    return [
        P("def clamp(value, low, high):\n    if value < low:\n        return low\n    if value > high:\n        return high\n"
          "    return value\n\ndef clamp_all(values, low, high):\n    out = []\n    for value in values:\n"
          "        out.append(clamp(value, low, high))\n    return out\n\ndef clamp_rows(rows, low, high):\n    out = []\n"
          "    for values in rows:\n        out.append(clamp_all(values, low, high))\n    return out\n",
          C, "nested helper functions", "loops that mirror the function above"),
        P("class Stack:\n    def __init__(self):\n        self.items = []\n\n    def push(self, item):\n        self.items.append(item)\n\n"
          "    def pop(self):\n        return self.items.pop()\n\n    def peek(self):\n        return self.items[-1]\n\n"
          "class Queue:\n    def __init__(self):\n        self.items = []\n\n    def push(self, item):\n        self.items.append(item)\n\n"
          "    def pop(self):\n        return self.items.pop(0)\n\n    def peek(self):\n        return self.items[0]\n",
          C, "two container classes", "second class repeats the first"),
        P("#include <stddef.h>\n\nfloat sum_f32(const float* x, size_t n) {\n    float acc = 0.0f;\n    for (size_t i = 0; i < n; ++i) acc += x[i];\n"
          "    return acc;\n}\n\ndouble sum_f64(const double* x, size_t n) {\n    double acc = 0.0;\n    for (size_t i = 0; i < n; ++i) acc += x[i];\n"
          "    return acc;\n}\n\nlong sum_i64(const long* x, size_t n) {\n    long acc = 0;\n    for (size_t i = 0; i < n; ++i) acc += x[i];\n    return acc;\n}\n",
          C, "C reductions per type", "type-parametric copies"),
        P("import unittest\n\nclass TestMath(unittest.TestCase):\n    def test_add(self):\n        self.assertEqual(add(1, 2), 3)\n\n"
          "    def test_sub(self):\n        self.assertEqual(sub(5, 2), 3)\n\n    def test_mul(self):\n        self.assertEqual(mul(3, 4), 12)\n\n"
          "    def test_div(self):\n        self.assertEqual(div(12, 4), 3)\n\n    def test_mod(self):\n        self.assertEqual(mod(7, 4), 3)\n",
          C, "unit-test boilerplate", "assertEqual lines"),
        P("SELECT id, name, email FROM users WHERE active = 1 ORDER BY name;\nSELECT id, name, email FROM admins WHERE active = 1 ORDER BY name;\n"
          "SELECT id, name, email FROM guests WHERE active = 1 ORDER BY name;\nSELECT id, name, email FROM vendors WHERE active = 1 ORDER BY name;\n"
          "SELECT id, name, email FROM partners WHERE active = 1 ORDER BY name;\n",
          C, "SQL statements differing by table", "same statement, other table"),
    ]


def _json_prompts() -> List[Prompt]:
    P, C = Prompt, PromptCategory.JSON
    return [
        P('{"users": [{"id": 1, "name": "Ada", "role": "admin", "active": true}, {"id": 2, "name": "Ben", "role": "user", "active": true}, '
          '{"id": 3, "name": "Cy", "role": "user", "active": false}, {"id": 4, "name": "Di", "role": "user", "active": true}, '
          '{"id": 5, "name": "Eli", "role": "admin", "active": true}]}',
          C, "array of records with one schema", "repeated keys"),
        P('{"config": {"server": {"host": "127.0.0.1", "port": 8080, "timeout_ms": 500}, "cache": {"host": "127.0.0.1", "port": 6379, '
          '"timeout_ms": 200}, "queue": {"host": "127.0.0.1", "port": 5672, "timeout_ms": 800}, "search": {"host": "127.0.0.1", "port": 9200, '
          '"timeout_ms": 900}}}',
          C, "nested service configuration", "host/port/timeout triples"),
        P('[{"t": "2024-01-01T00:00:00Z", "sensor": "a", "value": 20.5, "unit": "C"}, {"t": "2024-01-01T00:01:00Z", "sensor": "a", "value": 20.6, "unit": "C"}, '
          '{"t": "2024-01-01T00:02:00Z", "sensor": "a", "value": 20.6, "unit": "C"}, {"t": "2024-01-01T00:03:00Z", "sensor": "a", "value": 20.7, "unit": "C"}]',
          C, "time series", "timestamps advance by a minute"),
        P('{"openapi": "3.0.0", "paths": {"/items": {"get": {"summary": "List items", "responses": {"200": {"description": "OK"}}}, '
          '"post": {"summary": "Create item", "responses": {"201": {"description": "Created"}}}}, "/users": {"get": {"summary": "List users", '
          '"responses": {"200": {"description": "OK"}}}, "post": {"summary": "Create user", "responses": {"201": {"description": "Created"}}}}}}',
          C, "API description", "get/post blocks"),
        P('{"matrix": [[1, 0, 0, 0], [0, 1, 0, 0], [0, 0, 1, 0], [0, 0, 0, 1]], "inverse": [[1, 0, 0, 0], [0, 1, 0, 0], [0, 0, 1, 0], [0, 0, 0, 1]], '
          '"transpose": [[1, 0, 0, 0], [0, 1, 0, 0], [0, 0, 1, 0], [0, 0, 0, 1]]}',
          C, "numeric arrays", "identity rows"),
    ]


def _conversation_prompts() -> List[Prompt]:
    P, C = Prompt, PromptCategory.CONVERSATIONAL
    return [
        P("User: Can you explain what a cache line is?\nAssistant: A cache line is the unit of data moved between memory and the cache. "
          "When the processor reads one byte, the whole line that holds it is fetched.\nUser: How large is a cache line?\n"
          "Assistant: A cache line is usually 64 bytes on current processors, so reading one byte brings in the 63 bytes around it.\n"
          "User: Why does that matter for arrays?\nAssistant:",
          C, "technical question and answer", "answers reuse the question's wording"),
        P("User: I would like to book a table for two.\nAssistant: Of course. For which day would you like to book a table for two?\n"
          "User: Friday evening.\nAssistant: Friday evening works. At what time would you like the table for two on Friday evening?\n"
          "User: Seven o'clock.\nAssistant:",
          C, "booking dialogue", "confirmation echoes the request"),
        P("User: My build fails with an undefined reference to pthread_create.\nAssistant: An undefined reference to pthread_create means the "
          "thread library is not linked. Add -pthread to the link command.\nUser: Now it fails with an undefined reference to dlopen.\nAssistant:",
          C, "debugging help", "parallel answer structure"),
        P("User: Summarise the meeting.\nAssistant: The team agreed on three points. First, the release moves to next month. Second, the "
          "test plan is owned by the platform group. Third, the budget review happens before the release.\nUser: Repeat the second point.\nAssistant:",
          C, "summary then recall", "verbatim recall"),
        P("User: Translate 'good morning' to French.\nAssistant: 'Good morning' in French is 'bonjour'.\nUser: Translate 'good evening' to French.\n"
          "Assistant: 'Good evening' in French is 'bonsoir'.\nUser: Translate 'good night' to French.\nAssistant:",
          C, "translation drill", "template answers"),
    ]


def _repetitive_prompts() -> List[Prompt]:
    P, C = Prompt, PromptCategory.REPETITIVE
    return [
        P("one two three four five six seven eight nine ten " * 6, C, "counting loop", "exact period of ten words"),
        P("The quick brown fox jumps over the lazy dog. " * 8, C, "pangram repeated", "exact sentence repeats"),
        P("ABABABABABABABABABABABABABABABABABABABABABABABABABABABABABABABAB", C, "two-symbol alternation", "period two"),
        P("Row 1: ok\nRow 2: ok\nRow 3: ok\nRow 4: ok\nRow 5: ok\nRow 6: ok\nRow 7: ok\nRow 8: ok\nRow 9: ok\nRow 10: ok\nRow 11: ok\nRow 12: ok\n",
          C, "log lines with a counter", "only the number changes"),
        P("la la la, la la la, sing along with me; la la la, la la la, sing along with me; la la la, la la la, sing along with me; "
          "la la la, la la la, sing along with me; ", C, "chorus", "long exact period"),
    ]


class PromptDataset:
    def __init__(self, prompts: Optional[List[Prompt]] = None):
        self.prompts: List[Prompt] = list(prompts) if prompts is not None else []
        if prompts is None:
            self._initialize_default_prompts()

    def _initialize_default_prompts(self):
        self.prompts = _code_prompts() + _json_prompts() + _conversation_prompts() + _repetitive_prompts()

    def get_prompts(self, category: Optional[PromptCategory] = None) -> List[Prompt]:
        if category is None:
            return list(self.prompts)
        category = PromptCategory(category)
        return [p for p in self.prompts if p.category == category]

    def get_all_prompts(self) -> List[Prompt]:
        return list(self.prompts)

    def get_by_category_dict(self) -> Dict[str, List[Prompt]]:
        return {c.value: self.get_prompts(c) for c in PromptCategory}

    def add_prompt(self, prompt: Prompt):
        self.prompts.append(prompt)

    def to_dict(self) -> Dict[str, Any]:
        return {"categories": {c.value: [p.to_dict() for p in self.get_prompts(c)] for c in PromptCategory}}

    def to_json(self, indent: int = 2) -> str:
        return json.dumps(self.to_dict(), indent=indent)

    @classmethod
    def from_dict(cls, data: Dict[str, Any]) -> "PromptDataset":
        prompts: List[Prompt] = []
        for cat, items in data.get("categories", {}).items():
            for it in items:
                it = dict(it)
                it.setdefault("category", cat)
                prompts.append(Prompt.from_dict(it))
        return cls(prompts)

    @classmethod
    def from_file(cls, path: str) -> "PromptDataset":
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    def save_to_file(self, path: str):
        with open(path, "w", encoding="utf-8") as f:
            f.write(self.to_json())

    def __len__(self) -> int:
        return len(self.prompts)

    def __repr__(self) -> str:
        return "PromptDataset(" + ", ".join(f"{c.value}={len(self.get_prompts(c))}" for c in PromptCategory) + ")"


class TrainTestSplitter:
    """Cuts a text or a token sequence at `train_ratio`, moving the cut so that
    both parts keep their minimum length when the input is long enough."""

    def __init__(self, train_ratio: float = 0.6, min_train_length: int = 10, min_test_length: int = 5):
        if not 0.0 < train_ratio < 1.0:
            raise ValueError(f"train_ratio must be between 0 and 1, got {train_ratio}")
        self.train_ratio, self.min_train_length, self.min_test_length = train_ratio, min_train_length, min_test_length

    def _cut(self, n: int) -> int:
        cut = int(n * self.train_ratio)
        if n >= self.min_train_length + self.min_test_length:
            cut = min(max(cut, self.min_train_length), n - self.min_test_length)
        return max(0, min(cut, n))

    def split_text(self, text: str) -> Tuple[str, str]:
        c = self._cut(len(text))
        return text[:c], text[c:]

    def split_tokens(self, token_ids: List[int]) -> Tuple[List[int], List[int]]:
        c = self._cut(len(token_ids))
        return list(token_ids[:c]), list(token_ids[c:])

    def split(self, text: str, tokenizer=None) -> TrainTestSplit:
        if tokenizer is None:
            a, b = self.split_text(text)
            return TrainTestSplit(a, b)
        ids = list(tokenizer.encode(text))
        tr, te = self.split_tokens(ids)
        return TrainTestSplit(tokenizer.decode(tr), tokenizer.decode(te), tr, te)


class _CharTokenizer:
    vocab_size = 256

    def encode(self, text: str) -> List[int]:
        return list(text.encode("utf-8", errors="replace"))

    def decode(self, token_ids: List[int]) -> str:
        return bytes(int(t) & 0xFF for t in token_ids).decode("utf-8", errors="replace")


class TokenizerAdapter:
    """Uniform encode/decode over a Hugging Face tokenizer, anything with
    encode/decode, or the byte-level fall-back."""

    def __init__(self, tokenizer):
        self.tokenizer = tokenizer

    def encode(self, text: str) -> List[int]:
        out = self.tokenizer.encode(text)
        return list(out.ids) if hasattr(out, "ids") else list(out)

    def decode(self, token_ids: List[int]) -> str:
        return self.tokenizer.decode(list(token_ids))

    def encode_batch(self, texts: List[str]) -> List[List[int]]:
        return [self.encode(t) for t in texts]

    def get_vocab_size(self) -> int:
        for attr in ("vocab_size", "n_vocab"):
            v = getattr(self.tokenizer, attr, None)
            if v is not None:
                return int(v() if callable(v) else v)
        return len(self.tokenizer.get_vocab())

    @classmethod
    def create_char_level(cls) -> "TokenizerAdapter":
        return cls(_CharTokenizer())


DATA_FILE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "data", "test_prompts.json")


def get_default_dataset() -> PromptDataset:
    """The packaged JSON file when present, else the built-in prompts (they are the same set)."""
    if os.path.exists(DATA_FILE):
        return PromptDataset.from_file(DATA_FILE)
    return PromptDataset()


def get_prompts_by_category(category: str) -> List[Prompt]:
    return get_default_dataset().get_prompts(PromptCategory(category))


def create_splitter(train_ratio: float = 0.6) -> TrainTestSplitter:
    return TrainTestSplitter(train_ratio)


def get_char_level_tokenizer() -> TokenizerAdapter:
    return TokenizerAdapter.create_char_level()


def measure_ngram_acceptance(dataset: Optional[PromptDataset] = None, ngram_size: int = 3, max_draft_len: int = 5,
                             tokenizer: Optional[TokenizerAdapter] = None) -> Dict[str, float]:
    """Model-free acceptance estimate per category: build the cache from the
    train part, then walk the test part and count how many of the drafted tokens
    equal the true continuation (an upper bound for a model that reproduces the
    text)."""
    from .speculative import NgramCache
    dataset = dataset or get_default_dataset()
    tok = tokenizer or get_char_level_tokenizer()
    sp = TrainTestSplitter()
    out: Dict[str, float] = {}
    for cat in PromptCategory:
        drafted = accepted = 0
        for p in dataset.get_prompts(cat):
            tr, te = sp.split_tokens(tok.encode(p.text))
            cache = NgramCache(ngram_size)
            cache.build_from_sequence(tr)
            ctx = list(tr)
            i = 0
            while i < len(te):
                d = cache.draft_chain(ctx, max_draft_len)
                n = 0
                while n < len(d) and i + n < len(te) and d[n] == te[i + n]:
                    n += 1
                drafted += len(d)
                accepted += n
                step = te[i:i + n + 1]
                cache.update(step)
                ctx.extend(step)
                i += len(step)
        out[cat.value] = accepted / drafted if drafted else 0.0
    return out
