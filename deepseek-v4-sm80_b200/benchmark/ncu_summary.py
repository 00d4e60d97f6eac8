"""Per-kernel summary of an Nsight Compute launch list.

    ncu --metrics gpu__time_duration.sum --clock-control none -c N --csv --log-file launches.csv <program>
    python -m minisgl.benchmark.ncu_summary launches.csv [first-kernel-substring]

Groups the launches of the last step (from the last launch whose name contains the given substring, default
``embed``: the first kernel of a forward) by kernel and grid, and prints count, total and mean device time and the
share of the step.  The committed summaries under ``profiles/`` are made with it.
"""
import csv
import re
import sys

path = sys.argv[1]
first = sys.argv[2] if len(sys.argv) > 2 else 'embed'
with open(path) as f:
    lines=[l for l in f if not l.startswith('==')]
rows=[r for r in csv.DictReader(lines) if r.get('Metric Name')=='gpu__time_duration.sum']
names=[r['Kernel Name'] for r in rows]
idx=[i for i,n in enumerate(names) if first in n]
last=rows[idx[-1]:]
tot=sum(float(r['Metric Value'].replace(',','')) for r in last)
print("kernels in last step", len(last), "total us", tot/1000)
agg={}
for r in last:
    n=re.sub(r'\(.*','',r['Kernel Name']); n=re.sub(r'void |<unnamed>::','',n)
    key=(n[:44], r['Grid Size'])
    c,t=agg.get(key,(0,0)); agg[key]=(c+1,t+float(r['Metric Value'].replace(',','')))
for (n,g),(c,t) in sorted(agg.items(), key=lambda kv:-kv[1][1])[:45]:
    print(f"{n:44s} {g:>14s} x{c:3d} {t/1000:8.1f} us {100*t/tot:5.1f}%  avg {t/c/1000:6.1f}")
