"""Scrape configuration for the rollout exporters: written to the configured file, reload requested on the configured port."""
import yaml

from verl_b200.workers.rollout.metrics import prometheus_scrape_config, update_prometheus_config


def test_scrape_config_is_written_and_reload_requested(tmp_path):
    path = tmp_path / "prom" / "prometheus.yml"
    calls = []
    ok = update_prometheus_config({"file": str(path), "port": 9090}, ["10.0.0.1:9400", "10.0.0.2:9400"], "native", post=calls.append)
    assert ok and calls == ["http://127.0.0.1:9090/-/reload"]
    doc = yaml.safe_load(path.read_text())
    assert doc == prometheus_scrape_config(["10.0.0.1:9400", "10.0.0.2:9400"])
    assert doc["scrape_configs"][0]["static_configs"][0]["targets"] == ["10.0.0.1:9400", "10.0.0.2:9400"]
    assert not update_prometheus_config({"file": str(path), "port": 9090}, [], post=calls.append) and len(calls) == 1
    assert not update_prometheus_config({"port": 9090}, ["a:1"], post=calls.append)

    def refuse(url):
        raise OSError("connection refused")

    assert update_prometheus_config({"file": str(path), "port": 1}, ["a:1"], post=refuse)   # a host without Prometheus
