"""Monitor (metrics sink) configuration."""

from __future__ import annotations

from pathlib import Path

from .base import BaseConfig


class FileMonitorConfig(BaseConfig):
    path: Path | None = None          # file name/relative path of metrics.jsonl under <run_dir>/monitors/file
    compress_traces: bool = False
    trace_chunk_size: int = 256


class WandbMonitorConfig(BaseConfig):
    project: str = "prime-rl"
    entity: str | None = None
    name: str | None = None
    offline: bool = False
    log_samples: bool = False


class PrimeMonitorConfig(BaseConfig):
    base_url: str = "https://api.primeintellect.ai"
    api_key_var: str = "PRIME_API_KEY"
    run_name: str | None = None


class MonitorsConfig(BaseConfig):
    file: FileMonitorConfig | None = FileMonitorConfig()
    wandb: WandbMonitorConfig | None = None
    prime: PrimeMonitorConfig | None = None
