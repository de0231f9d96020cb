"""Tokenisers: a real ``tokenizer.json`` built in the test, the hash stand-in, padding rules."""
import pytest
import torch

from eridiffusion_b200.data.tokenizers import (HashTokenizer, HfTokenizer, TokenizerError, load_tokenizer,
                                               pad_or_truncate)


def _write_tokenizer(path):
    from tokenizers import Tokenizer, models, pre_tokenizers, processors
    vocab = {"<pad>": 0, "<s>": 1, "</s>": 2, "<unk>": 3, "a": 4, "photo": 5, "of": 6, "cat": 7, "dog": 8}
    tk = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tk.add_special_tokens(["<pad>", "<s>", "</s>", "<unk>"])
    tk.pre_tokenizer = pre_tokenizers.Whitespace()
    tk.post_processor = processors.TemplateProcessing(single="<s> $A </s>", special_tokens=[("<s>", 1), ("</s>", 2)])
    tk.save(str(path))


def test_hf_tokenizer_from_file_and_dir(tmp_path):
    f = tmp_path / "tokenizer.json"
    _write_tokenizer(f)
    for src in (str(f), str(tmp_path)):
        tok = HfTokenizer(src, max_length=8)
        ids, mask = tok(["a photo of a cat", "dog zebra"])
        assert ids.shape == (2, 8) and ids.dtype == torch.long
        assert ids[0].tolist() == [1, 4, 5, 6, 4, 7, 2, 0] and mask[0].tolist() == [True] * 7 + [False]
        assert ids[1].tolist()[:4] == [1, 8, 3, 2] and mask[1].sum() == 4
        assert tok.pad_id == 0 and tok.vocab_size == 9 and tok.decode(ids[0]) == "a photo of a cat"
    long_ids, m = HfTokenizer(str(f), max_length=4)("a photo of a cat")
    assert long_ids.shape == (1, 4) and m.all()
    with pytest.raises(TokenizerError):
        HfTokenizer(str(tmp_path / "missing.json"))


def test_hash_tokenizer_is_deterministic():
    tok = load_tokenizer(None, "clip")
    a, ma = tok("A photo, of a CAT")
    b, _ = tok(["a photo , of a cat"])
    assert torch.equal(a, b) and a.shape == (1, 77)
    assert a[0, 0] == 49406 and a[0, int(ma.sum()) - 1] == 49407 and ma.sum() == 8
    assert (a[0, 1:7] >= 1000).all() and (a[0, 1:7] < 49406 + 2).all()
    t5 = load_tokenizer("", "t5", max_length=16)
    ids, m = t5("hello world")
    assert ids.shape == (1, 16) and ids[0, 2] == 1 and ids[0, 3] == 0 and m.sum() == 3
    assert tok.word_id("cat") == HashTokenizer.clip().word_id("cat") != tok.word_id("dog")
    ids, n = pad_or_truncate(list(range(10)), 4, 0, eos_id=99)
    assert ids == [0, 1, 2, 99] and n == 4
    small = HashTokenizer(vocab_size=50, max_length=4)
    assert (small("x y")[0] < 50).all()


def test_verify_rms_norm_cli_passes(capsys):
    from eridiffusion_b200.cli.verify_rms_norm import main
    assert main(["--rows", "32", "--dim", "64", "--device", "cpu"]) == 0
    assert "7/7 passed" in capsys.readouterr().out
