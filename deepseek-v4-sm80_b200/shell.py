"""``python -m minisgl.shell``: interactive chat in the terminal against a locally spawned backend."""
from minisgl.server.launch import launch_server

if __name__ == "__main__":
    launch_server(run_shell=True)
