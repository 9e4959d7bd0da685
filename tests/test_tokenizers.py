"""Tokenizers and chat template (host side) on small vocabularies built here: no model vocabulary is shipped."""
import pytest

from slai_b200.tokenizers import (ChatTemplate, Gpt2Tokenizer, LlamaTokenizer, SPACE_MARK, bytes_to_unicode, split_pieces)


def llama_vocab():
    toks = ["<unk>", "<s>", "</s>"] + [f"<0x{b:02X}>" for b in range(256)]
    scores = [0.0] * len(toks)
    def add(t, s):
        toks.append(t)
        scores.append(s)
    for ch in "helowrd<>/s" + SPACE_MARK:
        add(ch, -100.0)
    add("he", -1.0); add("ll", -2.0); add("hell", -3.0); add("hello", -4.0); add(SPACE_MARK + "w", -5.0); add("or", -6.0)
    add(SPACE_MARK + "wor", -7.0); add("ld", -8.0); add(SPACE_MARK + "world", -9.0)
    return toks, scores


def test_llama_encode_merges_by_score_and_round_trips():
    toks, scores = llama_vocab()
    t = LlamaTokenizer(toks, scores)
    ids = t.encode("hello world", bos=True, eos=True)
    assert ids[0] == t.bos and ids[-1] == t.eos
    assert [toks[i] for i in ids[1:-1]] == ["hello", SPACE_MARK + "world"]
    assert t.decode_all(ids[1:-1]) == "hello world"
    # the best-scoring pair merges first: "he" (-1) before "ll" (-2), then "hell" (-3) needs "he"+"ll"
    assert [toks[i] for i in t.encode("hell", bos=False)] == ["hell"]


def test_llama_byte_fallback_and_special_strings():
    toks, scores = llama_vocab()
    t = LlamaTokenizer(toks, scores)
    ids = t.encode("é", bos=False)
    assert ids == [0xC3 + 3, 0xA9 + 3]                       # UTF-8 bytes of U+00E9 at id byte+3
    assert t.decode(-1, ids[0]) == chr(0xC3)                   # <0xC3> comes back as the single byte
    ids = t.encode("<s>hello</s>", bos=False)
    assert ids[0] == t.bos and ids[-1] == t.eos and [toks[i] for i in ids[1:-1]] == ["hello"]
    # right after BOS (id 1) leading white space of the piece is trimmed; U+2581 is not white space, so it survives the trim
    # and becomes a blank, exactly as `trim_start` then `replace` do in the reference
    assert t.decode(1, toks.index(SPACE_MARK + "world")) == " world"
    assert t.decode(5, toks.index(SPACE_MARK + "world")) == " world"
    t2 = LlamaTokenizer(toks + [" x"], scores + [0.0])
    assert t2.decode(1, len(toks)) == "x" and t2.decode(7, len(toks)) == " x"


def test_llama_from_gguf_metadata():
    toks, scores = llama_vocab()
    md = {"tokenizer.ggml.tokens": toks, "tokenizer.ggml.scores": scores, "tokenizer.ggml.bos_token_id": 1,
          "tokenizer.ggml.eos_token_id": 2, "tokenizer.ggml.unknown_token_id": 0}
    t = LlamaTokenizer.from_gguf(md)
    assert (t.bos_str(), t.eos_str(), t.unk) == ("<s>", "</s>", 0)


def test_byte_table_is_a_bijection_on_printable_characters():
    tab = bytes_to_unicode()
    assert len(tab) == 256 and len(set(tab.values())) == 256
    assert tab[ord("a")] == "a" and tab[ord(" ")] == chr(256 + 32) and tab[0] == chr(256)
    assert all(not c.isspace() for c in tab.values())


def test_split_pattern():
    assert split_pieces("Hello world, it's 42!") == ["Hello", " world", ",", " it", "'s", " 42", "!"]
    assert split_pieces("a  b") == ["a", " ", " b"] or split_pieces("a  b") == ["a", "  ", "b"]
    assert "".join(split_pieces("x\n\n y'll  ünï 7½")) == "x\n\n y'll  ünï 7½"


def gpt2_vocab():
    tab = bytes_to_unicode()
    base = [tab[b] for b in range(256)]
    sp = tab[ord(" ")]
    merges = ["h e", "l l", "he ll", "hell o", f"{sp} w", "o r", f"{sp}w or", "l d", f"{sp}wor ld"]
    toks = base + ["he", "ll", "hell", "hello", sp + "w", "or", sp + "wor", "ld", sp + "world", "<|endoftext|>"]
    return toks, merges


def test_gpt2_bpe_and_special_tokens():
    toks, merges = gpt2_vocab()
    eot = toks.index("<|endoftext|>")
    t = Gpt2Tokenizer(toks, merges, bos=eot, eos=eot)
    ids = t.encode("hello world<|endoftext|>hello")
    assert [toks[i] for i in ids] == ["hello", bytes_to_unicode()[32] + "world", "<|endoftext|>", "hello"]
    assert t.decode(ids[:2]) == "hello world"
    assert t.decode_bytes(t.encode("héllo")) == "héllo".encode("utf-8")     # bytes survive; decode() reads them as Latin-1
    assert t.bpe("hel") == ["he", "l"]
    with pytest.raises(KeyError):
        t.encode("<nope>")
    md = {"tokenizer.ggml.tokens": toks, "tokenizer.ggml.merges": merges, "tokenizer.ggml.bos_token_id": eot, "tokenizer.ggml.eos_token_id": eot}
    assert Gpt2Tokenizer.from_gguf(md).eos_str() == "<|endoftext|>"


def test_chat_template():
    pytest.importorskip("jinja2")
    msgs = [{"role": "system", "content": "Be brief."}, {"role": "user", "content": "Hi"}, {"role": "assistant", "content": "Hello."},
            {"role": "user", "content": "Bye"}]
    text = ChatTemplate.from_gguf({}).apply(msgs, "<s>", "</s>")
    assert text == "<s>[INST] <<SYS>>\nBe brief.\n<</SYS>>\n\nHi [/INST] Hello. </s><s>[INST] Bye [/INST]"
    custom = ChatTemplate("{% for m in messages %}{{ m['content'].split(' ')[-1] }};{% endfor %}{% if add_generation_prompt %}>{% endif %}{{ eos_token }}")
    assert "|split(" in custom.template and "|last" in custom.template
    assert custom.apply(msgs, "<s>", "</s>") == "brief.;Hi;Hello.;Bye;></s>"
    assert ChatTemplate.from_gguf({"tokenizer.chat_template": "{{ bos_token }}x"}).apply([], "B", "E") == "Bx"
