DEFAULT_METRICS_LOG_DIR = "/tmp/areno/tfevent"
