"""HfTokenizer and the incremental detokeniser against real `tokenizers` models trained in the test (byte-level
BPE, where a character can span tokens, and metaspace BPE, where the decoder strips the first token's space)."""
import random

import pytest

from ferrule_b200.utils.tokenizer import ByteTokenizer, HfTokenizer, IncrementalDecodeState, load_tokenizer

tokenizers = pytest.importorskip("tokenizers")

CORPUS = ["hello world, this is a test of the tokenizer", "héllo wörld – ünïcode ✓ 漢字 かな 🙂🙃",
          "def f(x):\n    return x + 1\n", "The quick brown fox jumps over the lazy dog. " * 3,
          "  leading spaces and\ttabs\n\nnewlines  "]


def _train(kind: str, directory) -> HfTokenizer:
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers
    if kind == "bytelevel":
        t = Tokenizer(models.BPE())
        t.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
        t.decoder = decoders.ByteLevel()
        tr = trainers.BpeTrainer(vocab_size=400, special_tokens=["<s>", "</s>"], show_progress=False,
                                 initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    else:
        t = Tokenizer(models.BPE(unk_token="<unk>"))
        t.pre_tokenizer = pre_tokenizers.Metaspace()
        t.decoder = decoders.Metaspace()
        tr = trainers.BpeTrainer(vocab_size=300, special_tokens=["<unk>", "<s>", "</s>"], show_progress=False)
    t.train_from_iterator(CORPUS, tr)
    t.save(str(directory / "tokenizer.json"))
    tok = load_tokenizer(directory)
    assert isinstance(tok, HfTokenizer)
    return tok


def _stream(tok, ids) -> str:
    st = IncrementalDecodeState(tok)
    return "".join(st.push(i) for i in ids) + st.finish()


def test_loader_falls_back_to_bytes_without_a_tokenizer_file(tmp_path):
    assert isinstance(load_tokenizer(tmp_path), ByteTokenizer)
    assert isinstance(load_tokenizer(None), ByteTokenizer)


@pytest.mark.parametrize("kind", ["bytelevel", "metaspace"])
def test_special_ids_and_round_trip(tmp_path, kind):
    tok = _train(kind, tmp_path)
    assert tok.bos_token_id >= 0 and tok.eos_token_id >= 0 and tok.bos_token_id != tok.eos_token_id
    ids = tok.encode("hello world", add_bos=True)
    assert ids[0] == tok.bos_token_id and tok.encode("hello world") == ids[1:]
    assert tok.decode(ids) == "hello world"                         # special tokens are skipped
    if kind == "bytelevel":
        for text in CORPUS:
            assert tok.decode(tok.encode(text)) == text


@pytest.mark.parametrize("kind", ["bytelevel", "metaspace"])
def test_streamed_text_equals_the_whole_decode(tmp_path, kind):
    tok = _train(kind, tmp_path)
    r = random.Random(0)
    texts = CORPUS + ["".join(r.choice("abc déf✓漢🙂 \n") for _ in range(60)) for _ in range(30)]
    for text in texts:
        ids = tok.encode(text)
        assert _stream(tok, ids) == tok.decode(ids)


@pytest.mark.parametrize("kind", ["bytelevel", "metaspace"])
def test_streamed_text_of_arbitrary_ids(tmp_path, kind):
    """Random ids: broken UTF-8 sequences and special tokens in mid-text.  The stream equals the whole decode up to
    a trailing incomplete character (which the stream drops)."""
    tok = _train(kind, tmp_path)
    r = random.Random(1)
    for _ in range(400):
        ids = [r.randrange(tok.vocab_size) for _ in range(r.randint(1, 40))]
        assert _stream(tok, ids) == tok.decode(ids).rstrip("�"), ids


def test_a_skipped_special_token_does_not_eat_the_next_space(tmp_path):
    tok = _train("metaspace", tmp_path)
    a, b = tok.encode("hello"), tok.encode("world")
    ids = a + [tok.eos_token_id] + b
    assert tok.decode(ids) == "hello world"
    assert _stream(tok, ids) == "hello world"
    assert _stream(tok, a + [tok.eos_token_id] * 3 + b) == "hello world"
