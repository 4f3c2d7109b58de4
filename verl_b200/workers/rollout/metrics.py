"""Prometheus export of the rollout engine's counters (``rollout.prometheus.enable`` / ``.port``): tokens prefilled and
generated, decode steps, time per phase, running / waiting requests and KV-block usage, one label set per replica.

Parity target: the reference's rollout servers export vLLM's Prometheus metrics when ``rollout.prometheus.enable`` is set
(``verl/trainer/config/rollout/rollout.yaml``, ``docs/advance/grafana_prometheus.md``).
"""

from __future__ import annotations

from typing import Optional

__all__ = ["RolloutMetricsExporter", "prometheus_scrape_config", "update_prometheus_config"]


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


def prometheus_scrape_config(server_addresses: list, scrape_interval: str = "10s") -> dict:
    """The Prometheus configuration that scrapes the given ``host:port`` exporters as job ``rollout``."""
    return {"global": {"scrape_interval": scrape_interval, "evaluation_interval": scrape_interval},
            "scrape_configs": [{"job_name": "rollout", "static_configs": [{"targets": [str(a) for a in server_addresses]}]}]}


def update_prometheus_config(config, server_addresses: list, rollout_name: Optional[str] = None, reload: bool = True,
                             post=None) -> bool:
    """Write the scrape configuration for the rollout exporters to ``config.file`` and ask a Prometheus server on this host
    (``config.port``) to reload it. Returns whether the file was written; a failed reload (no server on this host) is not
    an error, as on the nodes of a job that do not run Prometheus. ``post`` replaces the HTTP call in tests.

    Parity target: ``verl/workers/rollout/utils.py:141-223`` (which also copies the file to every node through Ray; here
    each host that calls this writes its own copy)."""
    import logging
    import os

    import yaml

    log = logging.getLogger(__name__)
    get = config.get if hasattr(config, "get") else (lambda k, d=None: getattr(config, k, d))
    if not server_addresses:
        log.warning("No server addresses available to update Prometheus config")
        return False
    path = get("file")
    if not path:
        return False
    try:
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(path, "w") as f:
            yaml.dump(prometheus_scrape_config(server_addresses), f, default_flow_style=False, indent=2)
        print(f"Updated Prometheus configuration at {path} with {len(server_addresses)} {(rollout_name or 'rollout').upper()} servers")
    except OSError as e:
        log.error("Failed to update Prometheus configuration: %s", e)
        return False
    if reload and get("port"):
        url = f"http://127.0.0.1:{int(get('port'))}/-/reload"
        try:
            if post is not None:
                post(url)
            else:
                import urllib.request

                urllib.request.urlopen(urllib.request.Request(url, method="POST"), timeout=5).close()
        except Exception:
            pass  # no Prometheus server on this host
    return True
