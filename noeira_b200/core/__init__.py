from .run import (CompositeLogger, CsvLogger, Logger, Metrics, NoOpLogger, PerfTimer, RemoteLogger, RunContext,  # noqa: F401
                  read_kv, write_kv)
