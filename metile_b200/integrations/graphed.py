"""One decode step of a patched model as a CUDA graph, replayed once per token.

Eager decoding of a patched model is bound by the interpreter, not by the GPU: a decoder block is
eleven kernels of a few microseconds each, and Python needs about 25 microseconds to issue one.  The
reference does not meet this problem (MLX evaluates a lazily built graph); here the equivalent is a
captured CUDA graph.  Every kernel of the patched decode step takes what changes from token to token
from device memory -- the token ids, the cache's per-sequence lengths (incremented on the device), the
cache rows themselves -- so one capture serves every later token.

    decoder = GraphedDecoder(model, batch=1, capacity=4096)       # inside apply_metile_to_torch_lm(...)
    logits = decoder.prefill(prompt_tokens)                       # eager
    tokens = decoder.generate(logits.argmax(-1), steps=128)       # graph replays, no host sync between

The model must offer `make_cache(batch, capacity)` returning `blocks.KVCache` objects and must run its
decode step through the patched path (the `attention` feature on, INT4 projections): a module that
falls back to its own forward slices the cache at the host's count, which a graph would freeze.
"""

from __future__ import annotations

import torch


def _logits_of(output):
    return getattr(output, "logits", output)


class GraphedDecoder:
    def __init__(self, model, batch=1, capacity=4096):
        self.model = model
        self.batch, self.capacity = int(batch), int(capacity)
        self.cache = model.make_cache(self.batch, self.capacity)
        device = self.cache[0].keys.device
        self.device = device
        self.token = torch.zeros((self.batch, 1), dtype=torch.long, device=device)   # input of the next step
        self.logits = None                                                          # output of the last step
        self.graph = None
        self.stream = torch.cuda.Stream(device)

    # ------------------------------------------------------------------------------------------
    def prefill(self, tokens):
        """Run the prompt [batch, length] eagerly through the model's own prefill path; returns the
        last position's logits [batch, vocabulary] (float32)."""
        if tokens.shape[0] != self.batch or tokens.shape[1] >= self.capacity:
            raise ValueError("prompt does not fit the decoder's batch or capacity")
        for cache in self.cache:
            cache.reset(0)
        with torch.no_grad():
            out = _logits_of(self.model(tokens, cache=self.cache))
        return out[:, -1, :].float()

    def _step(self):
        out = _logits_of(self.model(self.token, cache=self.cache))
        logits = out[:, -1, :].float()
        # The next step's input is chosen on the device: replays need no host in between.
        self.token.copy_(logits.argmax(dim=-1, keepdim=True))
        return logits

    def _capture(self):
        """Warm every lazily built piece on scratch caches, then capture one step on the real ones."""
        lengths = [cache.length for cache in self.cache]
        if min(lengths) < 1:
            raise ValueError("prefill before the first decode step")
        real, token = self.cache, self.token.clone()
        with torch.no_grad(), torch.cuda.stream(self.stream):
            self.stream.wait_stream(torch.cuda.current_stream(self.device))
            scratch = self.model.make_cache(self.batch, self.capacity)
            for cache, length in zip(scratch, lengths):
                cache.reset(length)
            self.cache = scratch
            self._step()                      # builds executors, fused q|k|v triples, workspaces
            self.cache = real
            self.token.copy_(token)
            self.stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=self.stream):
                self.logits = self._step()
            for cache, length in zip(self.cache, lengths):   # capture ran the host-side bookkeeping once
                cache.length = length
        torch.cuda.current_stream(self.device).wait_stream(self.stream)
        self.graph = graph

    def step(self, token=None):
        """One decode step.  `token` [batch] (long) overrides the device-side choice of the previous
        step.  Returns the logits buffer [batch, vocabulary] (overwritten by the next step)."""
        if token is not None:
            self.token.copy_(token.reshape(self.batch, 1))
        if self.graph is None:
            self._capture()
        if self.cache[0].length + 1 > self.capacity:
            raise ValueError("KV cache capacity exceeded")
        with torch.cuda.stream(self.stream):
            self.stream.wait_stream(torch.cuda.current_stream(self.device))
            self.graph.replay()
        torch.cuda.current_stream(self.device).wait_stream(self.stream)
        for cache in self.cache:
            cache.length += 1                 # the device-side count was advanced by the graph
        return self.logits

    def generate(self, first_token, steps):
        """Greedy decoding: `steps` graph replays fed by the device-side argmax; returns the generated
        tokens [batch, steps + 1] starting with `first_token`."""
        generated = [first_token.reshape(self.batch, 1).clone()]
        self.token.copy_(generated[0])
        for _ in range(steps):
            self.step()
            generated.append(self.token.clone())
        return torch.cat(generated, dim=1)
