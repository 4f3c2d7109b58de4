"""Prometheus export of the rollout engine's counters (``rollout.prometheus.enable`` / ``.port``): tokens prefilled and
generated, decode steps, time per phase, running / waiting requests and KV-block usage, one label set per replica.

Parity target: the reference's rollout servers export vLLM's Prometheus metrics when ``rollout.prometheus.enable`` is set
(``verl/trainer/config/rollout/rollout.yaml``, ``docs/advance/grafana_prometheus.md``).
"""

from __future__ import annotations

from typing import Optional

__all__ = ["RolloutMetricsExporter"]


class RolloutMetricsExporter:
    def __init__(self, replica: str = "0", registry=None, port: Optional[int] = None, namespace: str = "verl_rollout"):
        from prometheus_client import CollectorRegistry, Counter, Gauge, start_http_server

        self.registry = registry if registry is not None else CollectorRegistry()
        self.replica = str(replica)
        mk = lambda cls, name, doc: cls(f"{namespace}_{name}", doc, ["replica"], registry=self.registry)
        self.counters = {k: mk(Counter, k, d) for k, d in {
            "prefill_tokens": "prompt tokens run through the model", "prefill_tokens_shared": "prompt tokens served from a shared prefill",
            "generated_tokens": "tokens generated", "decode_steps": "decode steps executed",
            "prefill_seconds": "wall time spent in prefill", "decode_seconds": "wall time spent in decode"}.items()}
        self.gauges = {k: mk(Gauge, k, d) for k, d in {
            "running_requests": "requests holding a slot", "waiting_requests": "requests waiting for admission",
            "kv_blocks_free": "free KV-cache blocks", "kv_blocks_total": "KV-cache blocks", "kv_usage": "fraction of KV blocks in use"}.items()}
        self._last = {}
        if port:
            start_http_server(int(port), registry=self.registry)

    def update(self, engine) -> None:
        """Publish the engine's current counters (counters advance by the difference to the last call)."""
        st = dict(engine.stats)
        st["prefill_seconds"], st["decode_seconds"] = st.get("prefill_s", 0.0), st.get("decode_s", 0.0)
        for k, c in self.counters.items():
            now = float(st.get(k, 0.0))
            delta = now - self._last.get(k, 0.0)
            if delta > 0:
                c.labels(self.replica).inc(delta)
            self._last[k] = now
        total = int(getattr(engine, "num_blocks", 0) or 0)
        free = len(getattr(engine, "free_blocks", []))
        vals = {"running_requests": len(engine.running), "waiting_requests": len(engine.waiting), "kv_blocks_free": free,
                "kv_blocks_total": total, "kv_usage": (1.0 - free / total) if total else 0.0}
        for k, v in vals.items():
            self.gauges[k].labels(self.replica).set(v)
