"""Utilities: the typed-API name generator (``gen_api``), tracing / logging (``trace``), heap snapshots
(``checkpoint``) and roofline arithmetic (``roofline``)."""
