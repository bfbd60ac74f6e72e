#!/usr/bin/env bash
# PCIe ACS (Access Control Services) on PLX/PEX switches forces NIC<->GPU peer DMA through the root complex.
# The reference clears it before running with GPUDirect RDMA (scripts/disable_asc.sh:6-10, README.md:30-33).
# This script only LISTS the bridges it would touch unless --apply is given; it changes host PCIe state, needs
# root and setpci, and is never run by the library, the tests or the benchmarks.
set -euo pipefail
apply=0
[[ "${1:-}" == "--apply" ]] && apply=1
command -v lspci >/dev/null || { echo "lspci not found"; exit 1; }
mapfile -t bridges < <(lspci | grep -i -E "plx|pex|PCI bridge.*(Broadcom|PLX)" | awk '{print $1}')
if [[ ${#bridges[@]} -eq 0 ]]; then echo "no PLX/PEX bridges found: nothing to do"; exit 0; fi
for b in "${bridges[@]}"; do
  if [[ $apply -eq 1 ]]; then
    command -v setpci >/dev/null || { echo "setpci not found"; exit 1; }
    # ACS control register of the ACS extended capability: clear all enables
    setpci -s "$b" ECAP_ACS+6.w=0000 && echo "ACS cleared on $b"
  else
    echo "would clear ACS on $b (re-run with --apply as root)"
  fi
done
