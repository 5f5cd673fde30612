"""
``ios.draw`` placeholder.  The reference renders a graphviz PNG through ``pydot``
(``python/ios/visualizer.py:142``); plotting is not part of the execution path, so this build only
keeps the name importable and writes the textual schedule next to the requested file name.
"""


def draw(graph, fname, label=None):
    text = str(graph)
    with open(fname + '.txt', 'w') as f:
        if label:
            f.write(label + '\n')
        f.write(text + '\n')
    return fname + '.txt'
