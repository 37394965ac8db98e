"""The Python entry point: load a model folder and generate.

    from abacus_b200 import LM
    lm = LM("model_dir", dtype="bfloat16", max_tokens=65536)
    outs = lm.generate([[1, 2, 3], [4, 5]], max_new_tokens=32, temperature=0.0)

Option names and meanings follow abacus's command line (src/main.c:9-23): max_new_tokens is -n,
temperature is --temp (0 = greedy, default 0.7), seed is --seed (default: the time, src/main.c:112);
top_k is the 20 that src/main.c:41 fixes. Prompts are token-id lists, or strings when the folder has a tokenizer.json
(then raw=False wraps each in the chat template of src/main.c:168, as -p does, and raw=True
does not, as --raw).
"""
import os
import time

from .engine import Engine, load_model
from .engine.generate import Generator
from .sampling import Sampler

CHAT_TEMPLATE = "<|im_start|>user\n{}<|im_end|>\n<|im_start|>assistant\n<think>\n\n</think>\n\n"  # src/main.c:168
DEFAULT_CONTEXT = 4096   # abacus caps a sequence at 4,096 tokens (src/model.c:15)
DEFAULT_SEQUENCES = 8    # the cache's default room: this many sequences of that length


class LM:
    def __init__(self, folder, dtype="bfloat16", max_tokens=None, max_slots=None, max_context=None):
        self.model = load_model(folder, dtype)
        spec = self.model.spec
        if max_tokens is None:
            max_tokens = min(spec.max_positions, DEFAULT_CONTEXT) * DEFAULT_SEQUENCES
        self.engine = Engine(self.model, max_tokens=max_tokens, max_slots=max_slots, max_context=max_context)
        self.tokenizer = None
        if os.path.exists(os.path.join(folder, "tokenizer.json")):
            from .tokenizer import Tokenizer
            self.tokenizer = Tokenizer.from_file(os.path.join(folder, "tokenizer.json"))

    def stop_tokens(self):
        """<|im_end|> and <|endoftext|> when there is a tokenizer (src/main.c:176), and config.json's eos ids."""
        stops = set(self.model.spec.stop_tokens)
        if self.tokenizer is not None:
            stops.update(self.tokenizer.stop_ids())
        return sorted(stops)

    def encode(self, prompt, raw=False):
        if self.tokenizer is None:
            raise ValueError("this model folder has no tokenizer.json; give token ids")
        return self.tokenizer.encode(prompt if raw else CHAT_TEMPLATE.format(prompt))

    def generate(self, prompts, max_new_tokens=512, temperature=0.7, top_k=20, seed=None, stop_tokens=None,
                 batch_size=None, raw=False, return_requests=False, on_token=None):
        """Returns one list of new token ids per prompt (strings instead, if the prompts were strings).
        seed None: the time, as abacus's command line does; give a seed to draw the same tokens again.
        on_token(request, token) is called for every kept token as soon as the host has it."""
        if seed is None:
            seed = int(time.time())
        as_text = bool(prompts) and isinstance(prompts[0], str)
        ids = [self.encode(p, raw) for p in prompts] if as_text else [list(p) for p in prompts]
        sampler = Sampler(self.model.ctx.device, temperature=temperature, top_k=top_k, seed=seed)
        stops = self.stop_tokens() if stop_tokens is None else list(stop_tokens)
        gen = Generator(self.engine, sampler, stops, on_token=on_token)
        requests = gen.generate(ids, max_new_tokens, batch_size=batch_size)
        self.last_stats = gen.stats
        if return_requests:
            return requests
        if as_text:
            return [self.tokenizer.decode(r.output) for r in requests]
        return [r.output for r in requests]


def generate(folder, prompts, dtype="bfloat16", max_tokens=None, **options):
    """One call: load `folder` and generate for `prompts` (see LM.generate for the options)."""
    return LM(folder, dtype=dtype, max_tokens=max_tokens).generate(prompts, **options)
