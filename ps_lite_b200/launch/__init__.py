"""Job launchers: local processes, ssh, mpirun; all set the DMLC_* environment contract."""
