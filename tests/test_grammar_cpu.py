"""JSON-Schema-constrained decoding: schema subset, character matcher, token masks, generate hook.
Behaviours follow ferrotorch-grammar (schema.rs, state.rs, json_schema.rs)."""
import json

import pytest
import torch

from ferrotorch_b200.utils import grammar as G

PERSON = {"type": "object",
          "properties": {"name": {"type": "string", "minLength": 1, "maxLength": 5},
                         "age": {"type": "integer", "minimum": 0, "maximum": 150},
                         "tags": {"type": "array", "items": {"enum": ["a", "ab", 1, 12]}, "maxItems": 3},
                         "x": {"type": ["number", "null"]}, "ok": {"type": "boolean"}},
          "required": ["name", "age"]}


@pytest.mark.parametrize("text,want", [
    ('{"name":"bob","age":42}', True), ('{"age":42,"name":"bob"}', True),      # any key order
    ('{"name":"","age":1}', False), ('{"name":"toolong","age":1}', False),      # minLength / maxLength
    ('{"name":"b","age":151}', False), ('{"name":"b","age":-1}', False),        # maximum / minimum
    ('{"name":"b","age":150,"tags":["a","ab",12]}', True),                      # enum with shared prefixes
    ('{"name":"b","age":15,"tags":[1,1,1,1]}', False),                          # maxItems
    ('{"name":"b","age":1,"x":null,"ok":false}', True), ('{"name":"b","age":1,"x":-1.5e3}', True),
    ('{"name":"b"}', False),                                                    # required
    ('{"name":"b","age":1,"age":2}', False),                                    # a key only once
    ('{"name":"b","age":01}', False),                                           # no leading zeros
    ('{"name":"b\\u00e9\\n","age":7}', True), ('{"name":"b\\x","age":7}', False),   # escapes
    ('{"name":"b","age":1,"zz":1}', False),                                     # only listed properties
    ('{"name":"b","age":1.0}', False), ('{"name":"b","age":1e2}', False),       # integers are plain digits
    ('{ "name" : "b" ,\n "age" : 1 }', True),
])
def test_matcher_against_hand_checked_texts(text, want):
    assert G.validate(PERSON, text) is want
    if want:                                       # every accepted text is real JSON
        json.loads(text)


def test_whitespace_is_opt_in_and_next_chars():
    assert not G.validate(PERSON, '{ "name":"b","age":1}', whitespace_permissive=False)
    g = G.SchemaGrammar(PERSON)
    assert g.valid_next_chars() == ["{"] and not g.is_whitespace_permissive()
    g.step_text('{"')
    assert g.valid_next_chars() == ["a", "n", "o", "t", "x"]          # first letters of the five names
    g.step_text('age":1')
    assert "}" not in g.valid_next_chars() and "," in g.valid_next_chars()   # "name" is still owed
    with pytest.raises(G.GrammarError):
        g.step_char("}")
    g.step_text(',"name":"z"}')
    assert g.is_complete() and g.valid_next_chars() == []
    assert g.with_whitespace_permissive(True).is_whitespace_permissive()


def test_number_forms_and_constraints():
    num = {"type": "number"}
    for t, w in [("0", True), ("-0.5", True), ("1e5", True), ("-3.14E+2", True), ("0.5e-10", True), ("01", False),
                 ("1.", False), (".5", False), ("-", False), ("1e", False), ("+1", False), ("1e+", False)]:
        assert G.validate(num, t) is w, t
    assert G.validate({"type": "number", "multipleOf": 0.5}, "2.5") and not G.validate({"type": "number", "multipleOf": 0.5}, "2.4")
    assert G.validate({"type": "integer", "multipleOf": 3}, "12") and not G.validate({"type": "integer", "multipleOf": 3}, "13")
    g = G.SchemaGrammar({"type": "integer", "minimum": 5, "maximum": 99})
    g.step_text("12")
    assert g.is_complete() and g.valid_next_chars() == []             # a third digit cannot meet the bound
    g = G.SchemaGrammar({"type": "integer", "minimum": 0, "maximum": 150})
    g.step_text("15")
    assert g.valid_next_chars() == ["0"]                              # 151..159 could never be completed
    g = G.SchemaGrammar({"type": "integer", "minimum": -20, "maximum": -5})
    assert g.valid_next_chars() == ["-"]
    g.step_text("-")
    assert g.valid_next_chars() == ["1", "2", "5", "6", "7", "8", "9"]
    assert not G.SchemaGrammar({"type": "integer", "minimum": 1}).accepts("-")


def test_overlapping_alternatives_stay_alive():
    """Both branches start with a digit; the text decides later (the reference would commit to
    the first branch, schema.rs:33-41)."""
    s = {"oneOf": [{"type": "integer", "maximum": 5}, {"type": "number", "minimum": 2.5}]}
    assert G.validate(s, "3") and G.validate(s, "2.75") and G.validate(s, "7") and not G.validate(s, "2.25")
    s = {"anyOf": [{"type": "string", "maxLength": 2}, {"enum": ["hello"]}, {"type": "null"}]}
    assert G.validate(s, '"hi"') and G.validate(s, '"hello"') and G.validate(s, "null") and not G.validate(s, '"hey"')


def test_schema_subset_and_errors():
    s = {"type": "object", "properties": {"p": {"$ref": "#/$defs/point"}, "q": {"$ref": "#/definitions/flag"}},
         "required": ["p"], "$defs": {"point": {"type": "array", "items": {"type": "number"}, "minItems": 2, "maxItems": 2}},
         "definitions": {"flag": {"const": True}}, "title": "ignored", "additionalProperties": True}
    assert G.validate(s, '{"p":[1,2.5],"q":true}') and not G.validate(s, '{"p":[1]}') and not G.validate(s, '{"p":[1,2],"q":false}')
    for bad, msg in [({"allOf": [{"type": "string"}]}, "allOf"), ({"type": "string", "pattern": "a+"}, "pattern"),
                     ({"$ref": "#/$defs/a", "$defs": {"a": {"type": "array", "items": {"$ref": "#/$defs/a"}}}}, "recursive"),
                     ({"$ref": "http://x/y"}, "inside the document"), ({"$ref": "#/$defs/nope"}, "unresolvable"),
                     ({"type": "object", "properties": {}, "required": ["a"]}, "not declared"), ({"type": "tuple"}, "unsupported type"),
                     ({}, "without a type"), ({"enum": []}, "non-empty"), ({"type": "string", "minLength": 3, "maxLength": 1}, "maxLength"),
                     ({"type": "array"}, "needs items"), ("{oops", "not valid JSON")]:
        with pytest.raises(G.SchemaError, match=msg):
            G.Schema.from_json_schema(bad)
    assert isinstance(G.SchemaError("x"), ValueError)


VOCAB = ["<eos>", "{", "}", '"', ":", ",", "name", "age", '{"', '":', '","', "bob", "42", "4", "2", '"name"', '"age":',
         '":"', " ", "x", "na", "me", "ag", "e", "1500", "", '"}', "}x", "[", "]"]
SMALL = {"type": "object", "properties": {"name": {"type": "string", "maxLength": 8},
                                          "age": {"type": "integer", "minimum": 0, "maximum": 150}},
         "required": ["name", "age"]}


def test_token_masks_follow_the_characters():
    p = G.JsonSchemaProcessor(SMALL, VOCAB, eos_token_id=0)
    assert p.vocab_len() == len(VOCAB) and not p.is_complete()
    m = p.compute_mask()
    assert sorted(VOCAB[i] for i in m.allowed_ids()) == ["{", '{"'] and m.num_allowed() == 2
    assert m.packed().tolist() == [(1 << 1) | (1 << 8)]                # 32 ids per word, bit i = id i
    assert not m.is_allowed(0) and not m.is_allowed(VOCAB.index("")) and not m.is_allowed(10 ** 6)
    for piece in ['{"', "na", "me", '":"', "bob", '","', "age", '":', "4", "2"]:
        i = VOCAB.index(piece)
        assert p.compute_mask().is_allowed(i), piece
        p.step_token(i)
    m = p.compute_mask()
    assert not m.is_allowed(VOCAB.index("1500")) and not m.is_allowed(VOCAB.index("}x")) and m.is_allowed(VOCAB.index("}"))
    with pytest.raises(G.GrammarError):
        p.step_token(0)                                                # no end of sequence inside the object
    with pytest.raises(G.GrammarError):
        p.step_token(VOCAB.index("x"))
    p.step_token(VOCAB.index("}"))
    assert p.is_complete() and p.compute_mask().allowed_ids() == [0]
    p.step_token(0)
    logits = torch.zeros(2, len(VOCAB))
    out = p.compute_mask().apply(logits)
    assert out[0, 0] == 0 and torch.isinf(out[:, 1:]).all()
    assert G.TokenMask.allow_all(40).num_allowed() == 40 and G.TokenMask.allow_all(40).packed().tolist() == [-1, 255]


def test_mask_cache_counts_hits_by_state():
    p = G.JsonSchemaProcessor({"type": "array", "items": {"type": "string"}}, VOCAB, eos_token_id=0)
    cache = G.TokenTransitionCache()
    assert cache.is_empty()
    for t in ["[", '"', "bob", "x"]:
        p.compute_mask_cached(cache)
        p.step_token(VOCAB.index(t))
    p.compute_mask_cached(cache)          # still inside an unbounded string: same state as one step ago
    assert (cache.hits(), cache.misses(), len(cache)) == (2, 3, 3)
    a, b = p.compute_mask_cached(cache), p.compute_mask()
    assert torch.equal(a.bits, b.bits)
    cache.reset_counters()
    cache.clear()
    assert cache.hits() == 0 and cache.is_empty()


def test_generate_under_a_schema_yields_valid_json():
    from ferrotorch_b200.models.generation import GenerationConfig, generate
    from ferrotorch_b200.models.llama import LlamaConfig, LlamaForCausalLM
    pieces = ["<eos>"] + list('{}[]":,-.0123456789abcdefghijklmnopqrstuvwxyz ') + ['"name"', '"age"', "true", "false", "null", '":', '{"']
    torch.manual_seed(1)
    m = LlamaForCausalLM(LlamaConfig(vocab_size=len(pieces), hidden_size=32, intermediate_size=48, num_hidden_layers=1,
                                     num_attention_heads=2, num_key_value_heads=1)).eval()
    proc = G.SchemaLogitsProcessor(SMALL, pieces, eos_token_id=0)
    ids = torch.randint(1, len(pieces), (3, 4))
    cfg = GenerationConfig(max_new_tokens=80, temperature=1.0, do_sample=True, seed=3, eos_token_id=0)
    out = generate(m, ids, cfg, logits_processor=proc)
    done = 0
    for row in out[:, 4:].tolist():
        text = "".join(pieces[t] for t in row if t != 0)
        if 0 in row:                                  # finished rows are complete, valid values
            v = json.loads(text)
            assert set(v) == {"name", "age"} and 0 <= v["age"] <= 150 and len(v["name"]) <= 8
            done += 1
        else:                                         # the others are valid prefixes
            assert G.SchemaGrammar(SMALL).accepts(text)
    assert done >= 1 and proc.cache.hits() > 0


def test_native_mask_walk_equals_the_python_walk_and_is_shared():
    import random
    import string

    random.seed(1)
    vocab = ["<eos>", ""] + ["".join(random.choice(string.ascii_lowercase + string.digits + ' {}[]":,.-é\\') for _ in range(random.randint(1, 5)))
                            for _ in range(3000)] + ['"name"', '"age"', '":', '{"', '",', "}", ":"]
    nat = G.JsonSchemaProcessor(SMALL, vocab, eos_token_id=0, native=True)
    py = G.JsonSchemaProcessor(SMALL, vocab, eos_token_id=0, native=False)
    assert nat._native is not None and py._native is None
    for piece in ["", '{"', "name", '":"', "ab", '",', '"age"', ":", "15", "0", "}"]:
        if piece:
            nat.grammar().step_text(piece)
            py.grammar().step_text(piece)
        a, b = nat.compute_mask(), py.compute_mask()
        assert torch.equal(a.bits, b.bits), piece
    assert nat.is_complete() and nat.compute_mask().allowed_ids() == [0]
    st = nat._native.stats()
    assert st["trie_nodes"] > 3000 and st["transitions"] > 0 and st["states"] > 5
    twin = G.JsonSchemaProcessor(SMALL, vocab, eos_token_id=0, share=nat)           # a second row: same trie, same tables
    assert twin._native is nat._native and twin.vocab is nat.vocab
    assert torch.equal(twin.compute_mask().bits, G.JsonSchemaProcessor(SMALL, vocab, 0, native=False).compute_mask().bits)
    # an exception inside the matcher callback surfaces as a Python exception, not a crash
    broken = G.JsonSchemaProcessor({"type": "string"}, vocab, eos_token_id=0, native=True)
    broken.grammar()._m.step = lambda *_: (_ for _ in ()).throw(RuntimeError("boom"))
    broken.grammar()._memo.clear()
    with pytest.raises(RuntimeError, match="boom"):
        broken.compute_mask()


def test_packed_masks_round_trip_and_apply_in_place():
    torch.manual_seed(0)
    bits = torch.rand(3, 70) > 0.5
    packed = torch.stack([G.TokenMask(b).packed() for b in bits])
    assert packed.shape == (3, 3) and packed.dtype == torch.int32
    assert torch.equal(G.unpack_mask(packed, 70), bits)
    logits = torch.randn(3, 70)
    want = logits.masked_fill(~bits, float("-inf"))
    assert torch.equal(G.apply_packed_mask_(logits.clone(), packed), want)
    one = G.apply_packed_mask_(logits.clone(), packed[:1])                   # one mask row for every logits row
    assert torch.equal(one, logits.masked_fill(~bits[:1].expand(3, 70), float("-inf")))
    assert torch.equal(G.TokenMask(bits[0]).apply_(logits.clone()), one)
    for bad in (packed[:2], packed[:, :2]):
        with pytest.raises(ValueError):
            G.apply_packed_mask_(logits.clone(), bad)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_packed_mask_kernel_matches_torch(dtype):
    torch.manual_seed(0)
    bits = torch.rand(5, 128257) > 0.3
    packed = torch.stack([G.TokenMask(b).packed() for b in bits])
    logits = torch.randn(5, 128257, device="cuda").to(dtype)
    want = logits.masked_fill(~bits.cuda(), float("-inf"))
    assert torch.equal(G.apply_packed_mask_(logits.clone(), packed), want)
    assert torch.equal(G.apply_packed_mask_(logits.clone(), packed[:1]), logits.masked_fill(~bits[:1].cuda(), float("-inf")))


def test_reference_names_packed_vocab_masked_loop():
    from ferrotorch_b200 import models as M
    from ferrotorch_b200.utils import grammar as G

    vocab = ["<eos>", "{", "}", '"', "a", ":", "true", "false", "tr", "ue", ",", " ", '"a"', "1"]
    pv = G.PackedVocab.pack(vocab)
    assert len(pv) == len(vocab) and pv.max_token_len == 5 and pv.token(6) == "true" and pv.offsets[-1] == pv.chars.numel()
    assert G.JsonGrammar is G.SchemaGrammar
    st = G.BooleanEmissionStage.after("tr")
    assert st == G.BooleanEmissionStage.PartialTrue("ue") and st.allowed_next() == "u"
    assert G.BooleanEmissionStage.after("") is G.BooleanEmissionStage.Start and G.BooleanEmissionStage.Start.allowed_next() == "tf"
    assert G.BooleanEmissionStage.after("x") is None and G.BooleanEmissionStage.after("true") is None
    schema = {"type": "object", "properties": {"a": {"type": "boolean"}}, "required": ["a"]}
    proc = G.JsonSchemaProcessor(schema, vocab, 0)
    mask = G.compute_mask_gpu(proc, pv)
    assert mask.num_allowed() >= 1 and mask.is_allowed(1) and not mask.is_allowed(2)
    with pytest.raises(ValueError):
        G.compute_mask_gpu(proc, G.PackedVocab.pack(vocab[:3]))
    # greedy loop: the "model" prefers '}' everywhere; the grammar forces a valid document anyway
    logits = torch.zeros(len(vocab))
    logits[2], logits[7] = 5.0, 1.0
    out = M.masked_decode_loop(lambda ids: logits, proc, [], 32)
    text = "".join(vocab[i] for i in out)
    import json
    assert proc.is_complete() and isinstance(json.loads(text)["a"], bool)
    assert M.masked_decode_loop(lambda ids: logits, None, [1], 3) == [2, 2, 2]
    masked = M.apply_grammar_mask_gpu(torch.zeros(4), [True, False, True, False])
    assert masked.tolist() == [0.0, float("-inf"), 0.0, float("-inf")]
    q = M.GptqQ4(*__import__("ferrotorch_b200.serialize.quant_loaders", fromlist=["x"]).pack_gptq(torch.randn(16, 128), 128))
    assert (q.in_features, q.out_features) == (128, 16) and q.dequantize().shape == (16, 128)
    assert M.LlamaActivation.Silu == "silu" and M.LlamaMLP.__name__ == "SwiGLU"


# --------------------------------------------------------------------------- automaton walk over the whole vocabulary
def test_dfa_token_mask_equals_brute_force_and_the_schema_processor():
    import torch

    from ferrotorch_b200 import cubecl
    from ferrotorch_b200.utils.dfa_mask import DfaMaskInputs, compute_token_mask_dfa, literal_dfa
    from ferrotorch_b200.utils.grammar import JsonSchemaProcessor, PackedVocab

    vocab = ["t", "tr", "true", "rue", "e", "f", "false", "als", "alse", "x", "truex", "tru", "ue", "se", "fa", "T", "n", "null",
             "ull", "l", "u", "r", "a", "s", "", "é", "tré"]
    pv = PackedVocab.pack(vocab)
    for lits in (["true", "false"], ["null"], ["red", "rose", "ruse", "true"]):
        for emitted in ("", "t", "tr", "fal", "nul", "r", "ro", "true"):
            d = literal_dfa(lits, emitted)
            if d is None:
                assert not any(w.startswith(emitted) for w in lits)
                continue
            inp = DfaMaskInputs.new(d[0], d[1], pv.offsets, pv.chars, d[2], d[3], d[4], pv.max_token_len, vocab_size=len(vocab))
            got = compute_token_mask_dfa(inp)
            want = [bool(t) and any(w.startswith(emitted + t) for w in lits) for t in vocab]      # empty token: rejected
            assert got.tolist() == want, (lits, emitted)
    # the same masks as the general schema processor gives in its literal states
    plain = [t for t in vocab if t and t.isascii()]
    ppv = PackedVocab.pack(plain)
    for schema, lits in (({"type": "boolean"}, ["true", "false"]), ({"type": "null"}, ["null"])):
        for toks in ([], [lits[0][0]], [lits[0][0], lits[0][1]], [lits[-1][:2]] if lits[-1][:2] in plain else []):
            p = JsonSchemaProcessor(schema, plain)
            for t in toks:
                p.step_token(plain.index(t))
            d = literal_dfa(lits, "".join(toks))
            inp = DfaMaskInputs.new(d[0], d[1], ppv.offsets, ppv.chars, d[2], d[3], d[4], ppv.max_token_len)
            assert torch.equal(compute_token_mask_dfa(inp), p.compute_mask().bits), (schema, toks)
    # validation and the bounded loop
    d = literal_dfa(["true", "false"])
    assert DfaMaskInputs.new(d[0], d[1], pv.offsets[:-1], pv.chars, d[2], d[3], d[4], 5, vocab_size=len(vocab)) is None     # no sentinel
    assert DfaMaskInputs.new(d[0].reshape(-1)[:-1], d[1], pv.offsets, pv.chars, d[2], d[3], d[4], 5) is None                 # ragged table
    assert DfaMaskInputs.new(d[0], d[1], pv.offsets, pv.chars, d[2], 99, d[4], 5) is None                                    # bad start
    assert literal_dfa(["café"]) is None and literal_dfa([]) is None
    short = DfaMaskInputs.new(d[0], d[1], pv.offsets, pv.chars, d[2], d[3], d[4], 2)
    assert bool(compute_token_mask_dfa(short)[vocab.index("truex")])                 # walked two characters only, like the bounded kernel loop
    assert "vocab=%d" % len(vocab) in repr(short)
    assert cubecl.compute_token_mask_dfa_to_gpu is not None and cubecl.DfaMaskInputs is DfaMaskInputs
    assert torch.equal(cubecl.compute_token_mask_dfa_to_gpu(inp, device="cpu"), compute_token_mask_dfa(inp))
