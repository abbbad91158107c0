"""Region cache: exact memoisation and prefix reuse that always equals the whole tokenisation."""
import random
import re

from titanic_flash_41_b200.api.prompt_regions import RegionCache, cut_at

# a toy byte-level "BPE": pre-tokens are digit runs, letter runs with one leading space, or single other
# characters; every pre-token is cut into pieces of at most 3 characters.  Like the real tokenizer it has no
# look-behind and one character of look-ahead, so the safe-cut rule applies to it.
_PRE = re.compile(r"\d+| ?[A-Za-z]+|.", re.S)
_vocab, _rev = {}, []


def _id(piece):
    if piece not in _vocab:
        _vocab[piece] = len(_rev)
        _rev.append(piece)
    return _vocab[piece]


def encode(text):
    out = []
    for m in _PRE.finditer(text):
        s = m.group(0)
        out += [_id(s[i:i + 3]) for i in range(0, len(s), 3)]
    return out


def test_cut_rule():
    assert cut_at("a\nb", 2) and cut_at("ab12", 2) and cut_at("12ab", 2)
    assert not cut_at("abcd", 2) and not cut_at("a\n b", 2) and not cut_at("a\né", 2)


def test_exact_hits_and_prefix_reuse_equal_whole_tokenisation():
    rng = random.Random(0)
    words = ["alpha", "beta", "42", "gamma7", "x", "delta", "1999", "zeta"]
    doc = "\n".join(" ".join(rng.choice(words) for _ in range(rng.randint(3, 12))) for _ in range(400))
    calls = []

    def counted(t):
        calls.append(len(t))
        return encode(t)
    rc = RegionCache(counted, lambda i: _rev[i], min_chars=2000)
    first = doc + "\nQuestion one?"
    assert rc.tokens(first) == encode(first)
    assert rc.tokens(first) == encode(first) and rc.stats["hits"] == 1
    for q in ("\nQuestion two, with 123 numbers?", "\nAnother 9 8 7.", " trailing words only"):
        calls.clear()
        t = doc + q
        assert rc.tokens(t) == encode(t)
        assert max(calls) < len(t) // 4, "only the tail should have been tokenised"
    assert rc.stats["prefix_reuse"] == 3 and rc.stats["prefix_reuse_rejects"] == 0
    # an edit early in the document: no long common prefix -> whole tokenisation, still exact
    edited = "ZZ" + doc + "\nQ?"
    assert rc.tokens(edited) == encode(edited)
    # random edits at random places
    for _ in range(20):
        p = rng.randint(0, len(doc) - 1)
        t = doc[:p] + rng.choice(["7", " new", "\n", "x9"]) + doc[p:]
        assert rc.tokens(t) == encode(t)
    assert rc.stats["prefix_reuse_rejects"] == 0
    # capacity bound
    small = RegionCache(encode, lambda i: _rev[i], capacity_chars=len(doc) + 50, min_chars=2000)
    small.tokens(doc)
    small.tokens(doc + "x")
    assert len(small.items) == 1


def test_frontend_tokenises_through_the_region_cache():
    """The HTTP front end encodes the rendered chat marker by marker: the ids equal encoding the whole
    text, and a long document repeated in the next turn is served from the cache."""
    from titanic_flash_41_b200.api import protocol as P
    from titanic_flash_41_b200.api.server import Frontend
    from titanic_flash_41_b200.api.tokenizer import ByteTokenizer
    tok = ByteTokenizer(1024)
    f = Frontend(tok, 1 << 20)
    doc = "line of the document 12345\n" * 900
    body = {"messages": [{"role": "user", "content": doc + "first question"}], "max_tokens": 4}
    req, tokens, limit, pm = f.prepare(body)
    assert tokens == tok.encode(P.render_chat(req)) and pm is None
    body2 = {"messages": body["messages"] + [{"role": "assistant", "content": "answer"},
                                             {"role": "user", "content": "second question"}], "max_tokens": 4}
    req2, tokens2, _, _ = f.prepare(body2)
    assert tokens2 == tok.encode(P.render_chat(req2))
    assert f.regions.stats["hits"] >= 1                      # the document region was not tokenised again
