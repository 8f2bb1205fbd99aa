"""Decode under a JSON schema: whatever the (random, untrained) model prefers, every finished
sequence is a valid object of the schema.  Runs on CPU in a second."""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ferrotorch_b200.models.generation import GenerationConfig, generate  # noqa: E402
from ferrotorch_b200.models.llama import LlamaConfig, LlamaForCausalLM  # noqa: E402
from ferrotorch_b200.utils.grammar import JsonSchemaProcessor, SchemaLogitsProcessor  # noqa: E402

SCHEMA = {"type": "object",
          "properties": {"city": {"type": "string", "minLength": 1, "maxLength": 6},
                         "temp_c": {"type": "integer", "minimum": -40, "maximum": 50},
                         "sky": {"enum": ["clear", "cloudy", "rain"]}},
          "required": ["city", "temp_c", "sky"]}
# a toy vocabulary: single characters plus a few multi-character pieces, id 0 ends a sequence
VOCAB = ["<eos>"] + list('{}":,-_0123456789abcdefghijklmnopqrstuvwxyz') + ['"city"', '"temp_c"', '"sky"', '":', '{"', "clear", "cloudy", "rain"]


def main():
    torch.manual_seed(0)
    model = LlamaForCausalLM(LlamaConfig(vocab_size=len(VOCAB), hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                                         num_attention_heads=2, num_key_value_heads=1)).eval()
    proc = SchemaLogitsProcessor(SCHEMA, VOCAB, eos_token_id=0)
    prompt = torch.randint(1, len(VOCAB), (4, 3))
    cfg = GenerationConfig(max_new_tokens=96, temperature=1.0, do_sample=True, seed=1, eos_token_id=0)
    out = generate(model, prompt, cfg, logits_processor=proc)
    done = 0
    for row in out[:, 3:].tolist():
        text = "".join(VOCAB[t] for t in row if t != 0)
        if 0 in row:
            obj = json.loads(text)
            assert set(obj) == {"city", "temp_c", "sky"} and -40 <= obj["temp_c"] <= 50 and obj["sky"] in ("clear", "cloudy", "rain")
            done += 1
        print(text)
    print("finished %d of %d rows; mask cache: %d states, %d hits" % (done, out.shape[0], len(proc.cache), proc.cache.hits()))
    # the same machinery one token at a time
    p = JsonSchemaProcessor(SCHEMA, VOCAB, eos_token_id=0)
    print("first tokens allowed:", [VOCAB[i] for i in p.compute_mask().allowed_ids()])
    assert done >= 1


if __name__ == "__main__":
    main()
