"""StaticCache decode runtime for models whose Linear layers were swapped for the packed modules.

Mirrors ``ai_accel_lab/runtime_v5.py`` of the reference project: ``prepare_static_compile``
(:7-23) and ``generate_static_benchmark`` (:29-73, same timing protocol: warm-ups, one timed
prefill = TTFT, one timed fixed-length greedy generation, decode tok/s = generated /
(total - TTFT)).  These things differ:

* Token ids can be passed directly (``input_ids=``): the benchmark configurations use random
  prompts, and no tokenizer files are needed for them.
* ``StaticGraphDecoder`` is the native decode path: the one-token forward over a
  ``StaticCache`` is captured once into an explicit CUDA graph and replayed per token, instead of
  going through ``torch.compile(mode='reduce-overhead')``.  ``prepare_static_compile`` is kept
  for callers that want the reference's compiled path; the packed ops are registered custom ops
  with fake kernels, so Dynamo traces through them.
* Prompts that would need padding (a batch of texts of different lengths, or a length that is not
  a multiple of 8) are refused on the tokenizer path: the decoder keeps no attention mask, and
  attending to pad tokens would change the tokens and the TTFT.  Pass ``input_ids`` of equal length.
* ``decode_tokens_s`` / ``total_tokens_s`` are per sequence, as in the reference
  (generated / time); the whole-batch rates are reported as ``aggregate_decode_tokens_s`` /
  ``aggregate_total_tokens_s``.
* Under tensor parallelism the output projection can be split by vocabulary rows
  (``vocab_shard=(rank, world)``): every rank then holds ``vocab / world`` rows of ``lm_head``, and
  the greedy token is found with one small all-gather of each rank's (best logit, index) pair.
"""
from __future__ import annotations

import time

import torch


def prepare_static_compile(model, fullgraph=False):
    """Static KV cache + ``torch.compile(mode='reduce-overhead')`` on ``model.forward``.
    Returns ``(model, status)`` like the reference."""
    status = {"static_cache": False, "compiled": False, "graph_safe_custom_layers": 0, "error": None}
    try:
        for mod in model.modules():
            if hasattr(mod, "graph_safe"):
                mod.graph_safe = True
                status["graph_safe_custom_layers"] += 1
        if hasattr(model, "generation_config"):
            model.generation_config.cache_implementation = "static"
            status["static_cache"] = True
        model.forward = torch.compile(model.forward, mode="reduce-overhead", fullgraph=fullgraph)
        status["compiled"] = True
    except Exception as e:  # same soft-fail contract as the reference
        status["error"] = repr(e)
    return model, status


def compile_decoder_layers(model):
    """Fuse the element-wise work between the packed GEMVs (norms, rotary embedding, SwiGLU, residual
    adds) by compiling each decoder layer with Inductor -- regional compilation: all layers share one
    compiled artefact.  CUDA graphs stay explicit (StaticGraphDecoder.capture); the packed ops are
    opaque custom ops to the compiler."""
    layers = getattr(getattr(model, "model", model), "layers", None)
    if layers is None:
        raise ValueError("model has no .model.layers to compile")
    for layer in layers:
        if not getattr(layer, "_b200q_compiled", False):
            layer.forward = torch.compile(layer.forward, dynamic=False)
            layer._b200q_compiled = True
    return model


def _cuda_event_ms(fn):
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    r = fn()
    end.record()
    end.synchronize()
    return r, float(start.elapsed_time(end))


class StaticGraphDecoder:
    """Greedy decoding with a StaticCache and one captured CUDA graph for the decode step.

    ``prefill(input_ids)`` runs the prompt eagerly and returns the first generated token;
    ``decode(n)`` replays the captured single-token step ``n`` times with no host
    synchronisation in between and returns the ``[B, n]`` tokens.
    """

    def __init__(self, model, batch_size: int, max_cache_len: int, device=None, dtype=None, compile_layers=False,
                 vocab_shard=None, group=None, native_step=None):
        from transformers import StaticCache
        self.model = model
        # The decode step between the GEMVs: this package's kernels (decode_step.NativeDecodeStep) where the
        # model's architecture allows, else the framework's forward.  None = decide by the model.
        self.native = None
        self.native_reason = None
        self._want_native = native_step
        self.vocab_rank, self.vocab_world = vocab_shard if vocab_shard is not None else (0, 1)
        self.group = group
        if compile_layers:
            compile_decoder_layers(model)
        self.device = torch.device(device) if device is not None else next(model.parameters()).device
        self.batch = int(batch_size)
        self.max_len = int(max_cache_len)
        for mod in model.modules():
            if hasattr(mod, "graph_safe"):
                mod.graph_safe = True
        self.cache = StaticCache(config=model.config, max_cache_len=self.max_len)
        self.tok = torch.zeros((self.batch, 1), dtype=torch.long, device=self.device)
        self.pos = torch.zeros((1,), dtype=torch.long, device=self.device)
        self.graph = None
        self.out_tok = None

    def _greedy(self, last_logits: torch.Tensor) -> torch.Tensor:
        """Arg-max over the vocabulary, [B, V or V / world] -> [B, 1]; with a vocabulary-sharded output
        projection the ranks exchange their (best logit, global index) pairs."""
        if self.vocab_world <= 1:
            return last_logits.argmax(-1, keepdim=True)
        val, idx = last_logits.float().max(-1)
        mine = torch.stack([val, (idx + self.vocab_rank * last_logits.shape[-1]).float()], -1)      # [B, 2]; indices < 2^24 are exact
        flat = torch.empty((self.vocab_world * mine.shape[0], 2), dtype=mine.dtype, device=mine.device)
        torch.distributed.all_gather_into_tensor(flat, mine, group=self.group)
        every = flat.view(self.vocab_world, mine.shape[0], 2)
        best = every[..., 0].argmax(0)                                                               # first maximum: lowest rank, lowest index
        return every[best, torch.arange(mine.shape[0], device=mine.device), 1].long().unsqueeze(-1)

    def _bind_native(self):
        """After the first prefill (the cache allocates its tensors lazily): build the native decode step."""
        if self.native is not None or self._want_native is False or self.native_reason is not None:
            return
        from . import decode_step
        if self.device.type != "cuda":
            self.native_reason = "not a CUDA device"
        else:
            self.native_reason = decode_step.unsupported_reason(self.model)
        if self.native_reason is None:
            self.native = decode_step.NativeDecodeStep(self.model, self.cache, self.batch, self.max_len)
        elif self._want_native:
            raise NotImplementedError(f"native decode step: {self.native_reason}")

    @torch.no_grad()
    def _step(self):
        if self.native is not None:
            logits = self.native.step(self.tok, self.pos)
        else:
            out = self.model(input_ids=self.tok, past_key_values=self.cache, cache_position=self.pos, use_cache=True)
            logits = out.logits[:, -1]
        nxt = self._greedy(logits)
        self.tok.copy_(nxt)
        self.pos.add_(1)
        return nxt

    @torch.no_grad()
    def prefill(self, input_ids: torch.Tensor) -> torch.Tensor:
        b, n = input_ids.shape
        if b != self.batch or n >= self.max_len:
            raise ValueError("prompt does not fit the decoder's batch size / cache length")
        self.cache.reset()
        out = self.model(input_ids=input_ids, past_key_values=self.cache,
                         cache_position=torch.arange(n, device=self.device), use_cache=True)
        nxt = self._greedy(out.logits[:, -1])
        self.tok.copy_(nxt)
        self.pos.fill_(n)
        self._bind_native()
        return nxt

    @torch.no_grad()
    def capture(self):
        """Capture the decode step (call after a prefill; the cache contents are left intact
        apart from the warm-up positions, which the next prefill overwrites)."""
        if self.device.type != "cuda":
            raise RuntimeError("CUDA graphs need a CUDA device")
        saved_tok, saved_pos = self.tok.clone(), self.pos.clone()
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(2):
                self._step()
        torch.cuda.current_stream(self.device).wait_stream(side)
        self.tok.copy_(saved_tok)
        self.pos.copy_(saved_pos)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.out_tok = self._step()
        self.tok.copy_(saved_tok)
        self.pos.copy_(saved_pos)

    @torch.no_grad()
    def decode(self, n_tokens: int) -> torch.Tensor:
        if int(self.pos.item()) + n_tokens > self.max_len:
            raise ValueError("cache too short for the requested number of tokens")
        toks = torch.empty((self.batch, n_tokens), dtype=torch.long, device=self.device)
        for i in range(n_tokens):
            if self.graph is not None:
                self.graph.replay()
                toks[:, i:i + 1] = self.out_tok
            else:
                toks[:, i:i + 1] = self._step()
        return toks


@torch.no_grad()
def generate_static_benchmark(model, tokenizer=None, prompt=None, max_new_tokens=64, device="cuda", warmups=2,
                              input_ids=None, use_cuda_graph=True, compile_layers=False, vocab_shard=None, group=None,
                              native_step=None):
    """Fixed-length greedy generation benchmark (reference protocol, ai_accel_lab/runtime_v5.py:29-73).

    Either ``tokenizer`` + ``prompt`` (left-padded to a multiple of 8, as the reference does) or
    ``input_ids`` directly.  Returns a dict with the reference's keys (``ttft_ms``,
    ``decode_tokens_s``, ``total_tokens_s``, ``generated_tokens``, ``prompt_tokens``, memory
    figures) plus ``tokens`` (the generated ids)."""
    if input_ids is None:
        if tokenizer is None or prompt is None:
            raise ValueError("pass input_ids, or tokenizer and prompt")
        old = getattr(tokenizer, "padding_side", "right")
        tokenizer.padding_side = "left"
        if getattr(tokenizer, "pad_token_id", None) is None and getattr(tokenizer, "eos_token_id", None) is not None:
            tokenizer.pad_token_id = tokenizer.eos_token_id
        enc = tokenizer(prompt, return_tensors="pt", padding=True, pad_to_multiple_of=8)
        tokenizer.padding_side = old
        input_ids = enc["input_ids"]
        mask = enc.get("attention_mask") if hasattr(enc, "get") else None
        if mask is not None and not bool(mask.bool().all()):
            raise NotImplementedError("this prompt needs padding (left-padded to a multiple of 8): the static decoder keeps no "
                                      "attention mask, so pad tokens would be attended to; pass input_ids of equal length")
    input_ids = input_ids.to(device)
    b, n = input_ids.shape
    cuda = torch.device(device).type == "cuda"
    dec = StaticGraphDecoder(model, b, n + int(max_new_tokens) + 8, device=device, compile_layers=compile_layers,
                             vocab_shard=vocab_shard, group=group, native_step=False if compile_layers else native_step)

    for _ in range(max(1, int(warmups))):
        dec.prefill(input_ids)
    if cuda:
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        _, ttft = _cuda_event_ms(lambda: dec.prefill(input_ids))
    else:
        s = time.perf_counter()
        dec.prefill(input_ids)
        ttft = (time.perf_counter() - s) * 1000
    if cuda and use_cuda_graph:
        dec.capture()

    def run():
        first = dec.prefill(input_ids)
        rest = dec.decode(int(max_new_tokens) - 1)
        return torch.cat([first, rest], 1)

    for _ in range(max(1, int(warmups))):
        run()
    if cuda:
        torch.cuda.synchronize()
        out, total_ms = _cuda_event_ms(run)
        torch.cuda.synchronize()
    else:
        s = time.perf_counter()
        out = run()
        total_ms = (time.perf_counter() - s) * 1000
    generated = int(out.shape[1])
    decode_ms = max(0.001, total_ms - ttft)
    res = dict(prompt_tokens=n, generated_tokens=generated, ttft_ms=ttft,
               decode_tokens_s=generated / (decode_ms / 1000.0), total_tokens_s=generated / (total_ms / 1000.0),
               aggregate_decode_tokens_s=b * generated / (decode_ms / 1000.0),
               aggregate_total_tokens_s=b * generated / (total_ms / 1000.0),
               decode_ms_per_token=decode_ms / generated, batch=b, tokens=out, decoder=dec,
               decode_step="native" if dec.native is not None else f"framework ({dec.native_reason or 'native step not requested'})")
    if cuda:
        res.update(peak_vram_gb=torch.cuda.max_memory_allocated() / 1024 ** 3,
                   current_vram_gb=torch.cuda.memory_allocated() / 1024 ** 3,
                   reserved_vram_gb=torch.cuda.memory_reserved() / 1024 ** 3)
    return res
