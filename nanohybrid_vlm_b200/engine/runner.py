"""The model runner: the model, its cache and the one step function.

``step(items)`` runs exactly the tokens it is given, as one batch, from the cache that
earlier steps left, and returns fp32 logits at the wanted places.  Generation
(:mod:`.llm_engine`) and trace replay (``bin/trace_run``) both drive this object; neither
has a forward pass, a cache or a loader of its own.  The reference's counterpart is
nanovllm/engine/model_runner.py (init :39-258, cache sizing :650-916, run :2017-2058).
"""
from __future__ import annotations

import torch

from ..cache import CacheLayout, CacheManager, CacheStorage
from ..config import Config
from ..kernels import library, load_library, ops
from ..weights import load_weights, materialize_random
from .batch import BatchBuilder, StepItem
from .model import CausalLM


class InFlight:
    """A launched step: its chosen tokens are on the device (``device_tokens``: ``n`` tokens, then, at index
    ``width``, the step's health word; a captured graph's buffer is overwritten by the next replay of its bucket)
    and on their way to pinned host memory."""

    def __init__(self, n: int, width: int, device_tokens: torch.Tensor, slot):
        self.n, self.width, self.device_tokens, self._slot = n, width, device_tokens, slot

    def read(self) -> list[int]:
        """Wait for the step and return its tokens (raises ``KernelError`` if a bounded wait of a kernel ran out)."""
        buf, event = self._slot
        event.synchronize()
        host = buf[:self.width + 1].tolist()
        return ModelRunner._checked(host[:self.n] + host[-1:])


class ModelRunner:
    def __init__(self, config: Config, *, random_weights_seed: int | None = None, device: str = "cuda:0"):
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device: this engine computes on a B200 only and has no CPU fallback")
        load_library()   # compile / load the kernels now; fail loudly if that is impossible
        self.config = config
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.dtype = config.dtype
        spec = config.architecture.build_spec(config.model_config)
        self.model = CausalLM(spec, self.dtype, self.device)
        self.model.profile_ranges = bool(config.profile_ranges)
        if random_weights_seed is None:
            load_weights(self.model, config.model)
        else:
            materialize_random(self.model, random_weights_seed)
        self.vocab_size = spec.vocab_size
        self.decode_copy_bytes = self._prepare_decode_weights()

        self.layout = CacheLayout.from_needs(self.model.cache_needs())
        self.page_size = config.kvcache_block_size
        self.max_pages_per_seq = -(-config.max_model_len // self.page_size)
        num_slots = config.num_state_slots
        if num_slots < 0:
            num_slots = config.max_num_seqs if self.layout.needs_state_slots else 0
        num_pages = self._size_pools(num_slots)
        config.num_kvcache_blocks, config.num_state_slots = num_pages, num_slots
        counts = [num_pages] * len(self.layout.groups)
        possible = CacheManager.prefix_cache_possible(self.layout.groups, num_slots)
        if config.enable_prefix_cache and not possible:
            raise ValueError("enable_prefix_cache=True, but this model has layers with a window or with per-request "
                             "state, which shared pages cannot rebuild")
        config.enable_prefix_cache = possible if config.enable_prefix_cache is None else bool(config.enable_prefix_cache)
        self.cache = CacheManager(self.layout.groups, self.page_size, counts, num_slots,
                                  enable_prefix_cache=config.enable_prefix_cache)
        self.storage = CacheStorage(self.layout, spec.order, self.page_size, counts, num_slots, self.dtype, self.device,
                                    poison=config.poison_cache)
        self.builder = BatchBuilder(self.cache, self.vocab_size, self.device,
                                    max_tokens=config.max_num_batched_tokens, max_seqs=config.max_num_seqs,
                                    max_pages_per_seq=self.max_pages_per_seq, position_axes=spec.position_axes)
        # CUDA graphs of the decode step, one per batch-size bucket, captured at first use
        # (the reference captures the same buckets up front, nanovllm/engine/model_runner.py:2560-2594)
        self.graph_buckets = [] if config.enforce_eager else [b for b in (1, 2, 4, 8, 16, 32, 64, 128, 256, 512)
                                                             if b <= config.max_num_seqs]
        self._graphs: dict[int, tuple] = {}
        self._graph_pool = None
        self.last_logits: torch.Tensor | None = None    # fp32 logits of the last ``run`` (valid until the next one)
        widest = (self.graph_buckets[-1] if self.graph_buckets else 0) + 1
        self._host_tokens = [(torch.empty(widest, dtype=torch.int32, pin_memory=True), torch.cuda.Event()) for _ in range(2)]
        self._host_turn = 0

    def _prepare_decode_weights(self) -> int:
        """Second copies of the matrices that a decode step streams, laid out for the weight-streaming kernel
        (before the cache is sized, so that the pool gets what is left).  Returns the bytes they take."""
        cfg = self.config
        if self.dtype != torch.bfloat16 or cfg.decode_weight_copy is False:
            cfg.decode_weight_copy = False
            return 0
        weights = [(w, m) for w, m in self.model.streamed_weights() if ops.can_stream_slabs(w, m)]
        need = sum(ops.slab_copy_bytes(w, m) for w, m in weights)
        if cfg.decode_weight_copy is None:
            free, _ = torch.cuda.mem_get_info(self.device)
            cfg.decode_weight_copy = need <= free // 4
        if not cfg.decode_weight_copy:
            return 0
        ops.new_slab_family()            # this model's copies live and die together
        return sum(ops.prepare_streaming(w, m) for w, m in weights)

    # ------------------------------------------------------------------ sizing
    def _activation_allowance(self) -> int:
        """A generous bound on what one step's intermediate tensors take."""
        item = 2 if self.dtype == torch.bfloat16 else 4
        widest = max((d.shape[0] for bp in self.model.param_table() for d in [bp.decl] if len(d.shape) == 2
                      and d.shape[0] != self.vocab_size), default=self.model.spec.hidden_size)
        T = self.config.max_num_batched_tokens
        per_token = (3 * widest + 6 * self.model.spec.hidden_size) * item
        logits = self.config.max_num_seqs * self.vocab_size * (4 + item)
        return 2 * T * per_token + 2 * logits + (256 << 20)

    def _size_pools(self, num_slots: int) -> int:
        cfg = self.config
        per_page = sum(self.layout.page_bytes(self.page_size, self.dtype))
        useful = cfg.max_num_seqs * self.max_pages_per_seq       # more pages than this can never be held
        if cfg.num_kvcache_blocks > 0:
            return cfg.num_kvcache_blocks
        if per_page == 0:
            return 0
        free, total = torch.cuda.mem_get_info(self.device)
        used = total - free
        budget = int(total * cfg.gpu_memory_utilization) - used - self._activation_allowance()
        budget -= num_slots * self.layout.state_bytes_per_slot(self.dtype)
        pages = min(budget // per_page, useful)
        if pages < self.max_pages_per_seq:
            raise RuntimeError(f"not enough device memory for the cache: room for {max(pages, 0)} pages of "
                               f"{per_page} bytes, one request of max_model_len needs {self.max_pages_per_seq}")
        return int(pages)

    # ------------------------------------------------------------------ the step
    @torch.no_grad()
    def step(self, items: list[StepItem]) -> torch.Tensor:
        """Run the items' tokens as one batch; fp32 logits [number of wanted places, vocab] on the device,
        in the order of the items and of each item's ``want``."""
        batch = self.builder.build(items)
        return self.model.forward(batch, self.storage)

    @torch.no_grad()
    def run(self, items: list[StepItem], sampling) -> list[int]:
        """The step followed by the choice of one token per wanted row; host lists in, host list out.
        ``sampling``: (temperature, seed, position of the token being chosen) per wanted row.  A batch
        of single tokens replays the captured graph of its size bucket; anything else runs eagerly."""
        bucket = self._bucket(items)
        if bucket is None:
            batch = self.builder.build(items, sampling=sampling)
            logits = self.model.forward(batch, self.storage)
            out = torch.empty(batch.n_logit_rows + 1, dtype=torch.int32, device=self.device)   # tokens, health word
            ops.sample(out, logits, batch.temperatures, batch.seeds, batch.sample_positions)
            self.last_logits = logits
            return self._checked(out.tolist())
        if bucket not in self._graphs:
            self._capture(bucket)
        graph, tokens, launches, logits = self._graphs[bucket]
        self.builder.build(items, table_width=self.max_pages_per_seq, sampling=sampling, pad_to=bucket, views=False)
        graph.replay()
        library.LAUNCHES += launches     # the kernels that the replay launched
        self.last_logits = logits[:len(items)]
        host = tokens.tolist()           # one read: the bucket's tokens and the health word behind them
        return self._checked(host[:len(items)] + host[-1:])

    @staticmethod
    def _checked(tokens_and_health: list[int]) -> list[int]:
        """The step's tokens, if no bounded wait of a kernel ran out during the step (the health word that the
        sampler wrote behind the tokens is zero); else ``KernelError`` naming the kernel."""
        if tokens_and_health[-1] != 0:
            ops.raise_wait_errors()
        return tokens_and_health[:-1]

    def check_kernels(self) -> None:
        """For callers of ``step`` (logits, no sampler): raise ``KernelError`` if a bounded wait of a kernel ran
        out since the last check.  Synchronises the device."""
        ops.raise_wait_errors()

    # ------------------------------------------------------------------ a step whose tokens are read later
    @torch.no_grad()
    def launch(self, items: list[StepItem], sampling, feed_from: "InFlight | None" = None,
               feed: list[int] | None = None) -> "InFlight":
        """Start a step and return at once; ``InFlight.read()`` gives the tokens it chose, one per wanted row, later.
        ``feed_from`` / ``feed``: the step before it, still in flight, and per item the row of that step whose
        chosen token is the item's single token (-1: the item brings its own): such tokens are taken on the device
        (the values in the items are place-holders), so the host need not have read them.  A batch of single
        tokens replays the captured graph of its size bucket; anything else runs eagerly."""
        if feed_from is None:
            feed = None
        bucket = self._bucket(items)
        slot = self._host_tokens[self._host_turn]
        self._host_turn ^= 1
        if bucket is None:
            batch = self.builder.build(items, sampling=sampling, feed=feed)
            if feed is not None:
                ops.feed_tokens(batch.token_ids, self.builder.last_feed_src, feed_from.device_tokens, self.vocab_size)
            logits = self.model.forward(batch, self.storage)
            n = batch.n_logit_rows
            tokens = torch.empty(n + 1, dtype=torch.int32, device=self.device)      # tokens, health word
            ops.sample(tokens, logits, batch.temperatures, batch.seeds, batch.sample_positions)
            self.last_logits = logits
            if n + 1 > slot[0].numel():
                slot = (torch.empty(n + 1, dtype=torch.int32, pin_memory=True), slot[1])
            slot[0][:n + 1].copy_(tokens, non_blocking=True)
            slot[1].record()
            return InFlight(n, n, tokens, slot)
        if bucket not in self._graphs:
            self._capture(bucket)
        graph, tokens, launches, logits = self._graphs[bucket]
        n = len(items)
        self.builder.build(items, table_width=self.max_pages_per_seq, sampling=sampling, pad_to=bucket, views=False, feed=feed)
        if feed is not None:
            # between the host's copy of the batch arrays and the graph that reads them
            ops.feed_tokens(self.builder.last_token_ids, self.builder.last_feed_src, feed_from.device_tokens, self.vocab_size)
        graph.replay()
        library.LAUNCHES += launches
        self.last_logits = logits[:n]
        slot[0][:bucket + 1].copy_(tokens, non_blocking=True)     # tokens and health word, before the next replay overwrites them
        slot[1].record()
        return InFlight(n, bucket, tokens, slot)

    def _bucket(self, items) -> int | None:
        if not self.graph_buckets or len(items) > self.graph_buckets[-1]:
            return None
        if any(len(it.tokens) != 1 or it.want != [0] for it in items):
            return None
        return next(b for b in self.graph_buckets if b >= len(items))

    def _capture(self, bucket: int) -> None:
        """Capture model + sampler for `bucket` single-token requests.  The batch's device arrays live at
        fixed places of the builder's buffer for a given shape, so a replay reads what the next
        ``build`` of the same shape copied there."""
        def one_step():
            batch = self.builder.build([], table_width=self.max_pages_per_seq, sampling=[], pad_to=bucket)
            logits = self.model.forward(batch, self.storage)
            out = torch.empty(bucket + 1, dtype=torch.int32, device=self.device)
            ops.sample(out, logits, batch.temperatures, batch.seeds, batch.sample_positions)
            return out

        one_step()                       # warm up: library workspaces and kernel attributes are set outside capture
        torch.cuda.synchronize()
        batch = self.builder.build([], table_width=self.max_pages_per_seq, sampling=[], pad_to=bucket)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        launches_before = library.LAUNCHES
        with torch.cuda.graph(graph, pool=self._graph_pool):
            logits = self.model.forward(batch, self.storage)
            tokens = torch.empty(bucket + 1, dtype=torch.int32, device=self.device)     # tokens, health word
            ops.sample(tokens, logits, batch.temperatures, batch.seeds, batch.sample_positions)
        if self._graph_pool is None:
            self._graph_pool = graph.pool()
        self._graphs[bucket] = (graph, tokens, library.LAUNCHES - launches_before, logits)

    @torch.no_grad()
    def sample(self, logits: torch.Tensor, temperatures, seeds, positions) -> list[int]:
        """One token per logits row; host lists in, host list out."""
        n = logits.shape[0]
        dev = self.device
        t = torch.tensor(temperatures, dtype=torch.float32).pin_memory().to(dev, non_blocking=True)
        s = torch.tensor(seeds, dtype=torch.int64).pin_memory().to(dev, non_blocking=True)
        p = torch.tensor(positions, dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
        out = torch.empty(n, dtype=torch.int32, device=dev)
        ops.sample(out, logits, t, s, p)
        return out.tolist()
